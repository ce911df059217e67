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


def _failing_worker(rank, world, port, q, mode):
    """Step 1 is healthy.  Then rank 1 leaves between steps (`exit`) or stays but never joins the next gather
    (`silent`); rank 0 runs step 2 and must get ShardError, with its own slice attached, instead of hanging."""
    import datetime
    import time
    import torch.distributed as dist
    sys.path.insert(0, os.path.join(ROOT, "ppopp23-tdc_b200"))
    from tdc_b200.parallel import ShardError, forward_sharded
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    images = torch.arange(8.0).view(8, 1)
    out = forward_sharded(lambda x: x * 2, images)
    q.put((rank, "step1", out.flatten().tolist()))
    def leave():                            # flush the result queue, then go without tearing the broken group down
        q.close(); q.join_thread()
        os._exit(0)
    if rank == 1:
        if mode == "silent":
            time.sleep(12)                  # alive, but not in the collective: the group's timeout ends rank 0's wait
        leave()                             # between steps, nothing in flight
    t0 = time.time()
    try:
        forward_sharded(lambda x: x * 3, images)
        q.put((rank, "step2", "no error"))
    except ShardError as e:
        q.put((rank, "step2", ("ShardError", e.local.flatten().tolist(), time.time() - t0)))
    leave()


@pytest.mark.parametrize("mode", ["exit", "silent"])
def test_a_rank_that_leaves_between_steps_ends_the_next_gather_with_an_error(built, mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, port, q, mode)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=120) for _ in range(3)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    step1 = sorted(g for g in got if g[1] == "step1")
    assert [g[2] for g in step1] == [[2.0 * i for i in range(8)]] * 2
    (rank, _, res), = [g for g in got if g[1] == "step2"]
    assert rank == 0 and res[0] == "ShardError"
    assert res[1] == [3.0 * i for i in range(4)]          # rank 0's own slice was computed and is handed back
    assert res[2] < 60                                     # bounded: the connection error or the 4 s group timeout
