"""Batch sharding and the single gather, on CPU with gloo ranks (world size 2 and 3)."""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "ppopp23-tdc_b200"))


def test_shard_bounds_cover_the_batch(built):
    from tdc_b200.parallel import shard_bounds, shard_sizes
    for batch in (0, 1, 2, 7, 64, 255, 2048):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_bounds(batch, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == batch
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = shard_sizes(batch, world)
            assert sum(sizes) == batch and max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(8, 2, 2)


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def _worker(rank, world, port, batches, q):
    import torch.distributed as dist
    sys.path.insert(0, os.path.join(ROOT, "ppopp23-tdc_b200"))
    from tdc_b200.parallel import forward_sharded, shard_bounds
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        for batch in batches:
            g = torch.Generator().manual_seed(7)
            images = torch.randn(batch, 3, 4, 4, generator=g)            # same batch on every rank
            w = torch.randn(5, 3, 3, 3, generator=g)
            calls = []

            def forward(x):                                               # stand-in for the per-GPU forward
                calls.append(x.shape[0])
                return torch.nn.functional.conv2d(x, w, padding=1).mean((2, 3)) + 0.0 * rank

            out = forward_sharded(forward, images)
            q.put((batch, rank, out, calls, shard_bounds(batch, world, rank)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,batches", [(2, (8, 7, 1)), (3, (4,))])
def test_sharded_forward_equals_single_process(built, world, batches):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, batches, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in range(world * len(batches))]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for batch, rank, out, calls, (a, b) in results:
        g = torch.Generator().manual_seed(7)
        images = torch.randn(batch, 3, 4, 4, generator=g)
        w = torch.randn(5, 3, 3, 3, generator=g)
        whole = torch.nn.functional.conv2d(images, w, padding=1).mean((2, 3))
        assert out.shape == whole.shape
        assert torch.allclose(out, whole, atol=1e-6)      # every rank holds the full result, rank order kept
        assert calls == ([b - a] if b > a else [1])       # one forward on its slice (one image if it owns none)
