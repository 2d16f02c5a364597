"""Host-side multi-rank logic on CPU: two gloo ranks shard a batch, plan identical replicas (dry run,
no device), gather ragged outputs in image order and agree on the max of their timings."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_bounds_partition_the_batch():
    from deepracin_b200 import replicas
    for batch in (0, 1, 7, 64, 129):
        for world in (1, 2, 3, 8):
            spans = [replicas.shard_bounds(batch, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == batch
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        replicas.shard_bounds(8, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import deepracin_b200 as dr
    import nets
    from deepracin_b200 import replicas
    dist = replicas.init("gloo")
    images = nets.synthetic_images("replica_test", 5, 32)            # 5 images over 2 ranks: ragged shards 3 + 2
    mine = replicas.shard(images, world, rank)
    # every rank plans its own replica of the same graph for its own slice (no device: dry run)
    with dr.Environment() as env:
        g = env.create_graph("HWC")
        g.batch = mine.shape[0]
        x, out = nets.squeezenet11(g, size=32, classes=16)
        dr.mark_as_output(out)
        dr.lib.dR_setDryRun(g.ptr, 1)
        dr.lib.dR_setBatchSize(g.ptr, g.batch)
        assert dr.lib.dR_prepare(g.ptr)
        order = [dr.lib.dR_getScheduledNodeId(g.ptr, i) for i in range(dr.lib.dR_getScheduleLength(g.ptr))]
        nbuf = dr.lib.dR_getStreamBufferCount(g.ptr)
    # stand-in for the per-image outputs: each image's mean, so order and raggedness are checkable
    local = mine.reshape(mine.shape[0], -1).mean(1, keepdims=True).astype(np.float32)
    allout = replicas.gather_outputs(dist, local, images.shape[0])
    tmax = replicas.max_over_ranks(dist, 10.0 + rank)
    replicas.barrier(dist)
    q.put((rank, mine.shape[0], order, nbuf, allout, tmax))
    replicas.finish(dist)


def test_two_gloo_ranks_shard_plan_and_gather():
    import torch.multiprocessing as mp
    import nets
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=180) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (r0, n0, order0, nbuf0, out0, t0), (r1, n1, order1, nbuf1, out1, t1) = res
    assert (n0, n1) == (3, 2)
    assert order0 == order1 and nbuf0 == nbuf1               # identical replicas
    want = nets.synthetic_images("replica_test", 5, 32).reshape(5, -1).mean(1, keepdims=True)
    assert np.allclose(out0, want) and np.array_equal(out0, out1)
    assert t0 == t1 == 11.0
