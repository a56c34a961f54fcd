"""The multi-rank path on CPU: two gloo ranks each take a batch shard, run the forward on
their shard (here through the CPU checker, standing in for the GPU kernel) and the gathered
result must equal the unsharded forward.  No collective is on the data path; the gather is
for checking only, as in the benchmark."""
import os
import socket
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(('127.0.0.1', 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, n_total, q):
    sys.path.insert(0, ROOT)
    import oracle
    from mmcv_b200.shard import batch_shard
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(n_total, 8, 9, 7, generator=gen)
    off = torch.randn(n_total, 2 * 18, 9, 7, generator=gen) * 2
    msk = torch.sigmoid(torch.randn(n_total, 2 * 9, 9, 7, generator=gen))
    w = torch.randn(6, 8, 3, 3, generator=gen) * 0.1
    b = torch.randn(6, generator=gen)
    n0, n1 = batch_shard(n_total, rank, world)
    part = oracle.port_forward(x[n0:n1], off[n0:n1], msk[n0:n1], w, b, 1, 1, 1, 1, 2)
    per = (n_total + world - 1) // world
    padded = torch.zeros(per, *part.shape[1:])
    padded[:n1 - n0] = part
    parts = [torch.zeros_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded)
    # max-over-ranks reduction as the benchmark does for its timing
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        full = oracle.port_forward(x, off, msk, w, b, 1, 1, 1, 1, 2)
        got = torch.cat(parts)[:n_total]
        q.put((torch.equal(got, full), t.item()))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_batch_shards_reassemble():
    ctx = mp.get_context('spawn')
    for n_total in (4, 5):          # even split and ragged last shard
        q = ctx.Queue()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, 2, port, n_total, q)) for r in range(2)]
        for p in procs:
            p.start()
        ok, mx = q.get(timeout=120)
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
        assert ok and mx == 2.0


def test_batch_shard_covers_everything_once():
    from mmcv_b200.shard import batch_shard
    for n in (0, 1, 7, 256):
        for world in (1, 2, 4, 8):
            seen = []
            for r in range(world):
                a, b = batch_shard(n, r, world)
                seen += list(range(a, b))
            assert seen == list(range(n))
