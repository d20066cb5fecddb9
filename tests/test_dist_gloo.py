"""Host logic of the multi-GPU path on CPU: batch sharding and the single filter-gradient
all-reduce, as two gloo ranks."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from portdnn_b200 import dist as pdist  # noqa: E402


def test_shard_batch_covers_the_batch_once():
    for batch in (1, 7, 256, 2048, 2050):
        for world in (1, 2, 4, 8):
            spans = [pdist.shard_batch(batch, world, r) for r in range(world)]
            assert spans[0][0] == 0
            assert sum(c for _, c in spans) == batch
            for (s0, c0), (s1, _) in zip(spans, spans[1:]):
                assert s0 + c0 == s1
            assert max(c for _, c in spans) - min(c for _, c in spans) <= 1
    with pytest.raises(ValueError):
        pdist.shard_batch(8, 2, 2)


def test_gradient_layout_is_aligned_and_padded():
    offsets, total = pdist.filter_gradient_layout([9408, 4096, 36864, 10], pad_to=100000)
    assert offsets == [0, 9408, 13504, 50368]
    assert all(o % 64 == 0 for o in offsets)
    assert total == 100000


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # each rank computes the filter gradient of its shard of a tiny convolution on the CPU
        # oracle; the all-reduced bucket must equal the gradient of the whole batch
        from oracle import oracle as orc
        rng = np.random.default_rng(5)
        n, h, w, c, k = 6, 5, 5, 3, 4
        p_all = orc.conv_params(n, h, w, c, k, 3, 1, True)
        x = rng.standard_normal(n * h * w * c).astype(np.float32)
        dy = rng.standard_normal(n * h * w * k).astype(np.float32)
        start, count = pdist.shard_batch(n, world, rank)
        p = orc.conv_params(count, h, w, c, k, 3, 1, True)
        xs = x.reshape(n, -1)[start:start + count].ravel()
        dys = dy.reshape(n, -1)[start:start + count].ravel()
        bucket = pdist.FilterGradientBucket([9 * c * k, 5], "cpu", pad_to=256)
        bucket.view(0).copy_(torch.from_numpy(orc.conv2d(orc.FILTER_BACKPROP, xs, dys, p)))
        bucket.view(1).fill_(float(rank + 1))
        bucket.all_reduce()
        ref = orc.conv2d(orc.FILTER_BACKPROP, x, dy, p_all)
        ok = np.allclose(bucket.view(0).numpy(), ref, rtol=1e-5, atol=1e-5)
        ok = ok and bucket.view(1).tolist() == [float(sum(range(1, world + 1)))] * 5
        slowest = pdist.max_over_ranks(10.0 + rank)
        ok = ok and slowest == 10.0 + world - 1
        out[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_two_ranks_sum_their_filter_gradients():
    world = 2
    from oracle import oracle as orc
    orc.build()
    mgr = mp.Manager()
    out = mgr.dict()
    port = 29000 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    assert dict(out) == {0: True, 1: True}


def _failing_worker(rank, world, port, out, mode):
    """Host-injected failures: rank 1 raises in its backward pass ("raise") or leaves without a word
    ("silent"); rank 0 must get RankFailure before the collective instead of blocking in it."""
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    store = dist.TCPStore("127.0.0.1", port + 1, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=20))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        guard = pdist.StepGuard(store, rank, world, timeout_s=2.0)
        bucket = pdist.FilterGradientBucket([8], "cpu")

        def backward():
            if rank == 1 and mode == "raise":
                raise ValueError("injected")
            bucket.view(0).fill_(1.0)

        # step 0 goes through on both ranks
        guard.guarded_all_reduce(bucket, 0, lambda: bucket.view(0).fill_(float(rank + 1)))
        step0_ok = bucket.view(0).tolist() == [3.0] * 8
        if rank == 1 and mode == "silent":
            out[rank] = ("left", step0_ok)
            return
        try:
            guard.guarded_all_reduce(bucket, 1, backward)
            out[rank] = ("no error", step0_ok)
        except pdist.RankFailure as e:
            out[rank] = ("RankFailure", step0_ok, str(e))
        except ValueError:
            out[rank] = ("raised", step0_ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["raise", "silent"])
def test_a_failed_rank_is_noticed_before_the_collective(mode):
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    port = 31000 + (os.getpid() % 2000) + (0 if mode == "raise" else 7)
    mp.spawn(_failing_worker, args=(world, port, out, mode), nprocs=world, join=True)
    res = dict(out)
    assert res[0][0] == "RankFailure" and res[0][1], res
    assert res[1][0] == ("raised" if mode == "raise" else "left") and res[1][1], res
    assert ("rank 1" in res[0][2]), res
