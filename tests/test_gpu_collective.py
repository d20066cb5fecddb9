"""The library's own collective (pdnn_comm_* / pdnn_allreduce_filter_grads) on two GPUs: each rank runs
the filter backprop of its shard of the batch through the C ABI, the gradients are summed over ranks,
and the sum equals the oracle's gradient of the whole batch.  One process per GPU; the 128-byte
communicator id travels through a TCP store.  NVLS is off, as for every test that ends ranks."""
import datetime
import os
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, out):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    from oracle import oracle as orc
    import portdnn_b200 as pd
    from portdnn_b200 import dist as pdist
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=60))

    def exchange(ident):
        if ident is not None:
            store.set("pdnn_comm_id", ident)
        return store.get("pdnn_comm_id")

    comm = pdist.GradientComm(rank, world, exchange)
    try:
        rng = np.random.default_rng(11)
        n, h, w, c, k = 8, 14, 14, 64, 128
        x = rng.standard_normal(n * h * w * c).astype(np.float32)
        dy = rng.standard_normal(n * h * w * k).astype(np.float32)
        start, count = pdist.shard_batch(n, world, rank)
        p = pd.conv_params(count, h, w, c, k, 3, 1)
        xs = torch.from_numpy(x.reshape(n, -1)[start:start + count].ravel().copy()).to(device).to(torch.bfloat16)
        dys = torch.from_numpy(dy.reshape(n, -1)[start:start + count].ravel().copy()).to(device).to(torch.bfloat16)
        bucket = pdist.FilterGradientBucket([9 * c * k, 5], device)
        pd.conv2d(pd.FILTER_BACKPROP, xs, dys, p, out=bucket.view(0), output_f32=True)
        bucket.view(1).fill_(float(rank + 1))
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):  # the stage's span on its own stream, as the training step does
            bucket.all_reduce(span=bucket.span(0, 0), comm=comm)
        bucket.all_reduce(span=bucket.span(1, 1), comm=comm)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        got = bucket.view(0).cpu().numpy()
        p_all = orc.conv_params(n, h, w, c, k, 3, 1, True)
        xq = torch.from_numpy(x).to(torch.bfloat16).float().numpy()
        dq = torch.from_numpy(dy).to(torch.bfloat16).float().numpy()
        ref = orc.conv2d(orc.FILTER_BACKPROP, xq, dq, p_all)
        err = float(np.abs(got - ref).max() / np.abs(ref).max())
        out[rank] = (err, bucket.view(1).tolist(), pd.device_error_record()[0])
    finally:
        comm.destroy()


def test_two_gpus_sum_their_filter_gradients_through_the_c_abi():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from oracle import oracle as orc
    from portdnn_b200 import build
    orc.build()
    build.build()
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    port = 33000 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    res = dict(out)
    assert set(res) == {0, 1}
    for rank in range(world):
        err, ones, record = res[rank]
        assert err < 1e-4, res  # fp32 accumulation of exactly-representable bf16 products
        assert ones == [3.0] * 5
        assert record == 0


def test_collective_rejects_bad_arguments_without_a_communicator():
    import ctypes
    import portdnn_b200 as pd
    L = pd.api.lib()
    buf = torch.zeros(8, device="cuda")
    assert L.pdnn_allreduce_filter_grads(None, ctypes.c_void_p(buf.data_ptr()), ctypes.c_size_t(8), None) == int(pd.api.StatusCode.InvalidParameter)
    assert L.pdnn_allreduce_filter_grads(None, None, ctypes.c_size_t(0), None) == 0  # nothing to sum
    comm = ctypes.c_void_p()
    assert L.pdnn_comm_init(ctypes.byref(comm), bytes(128), 2, 2) == int(pd.api.StatusCode.InvalidParameter)
    assert L.pdnn_comm_destroy(None) == 0
