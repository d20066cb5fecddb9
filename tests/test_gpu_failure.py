"""Failure detection of the tensor-core kernels without a fault: every barrier wait in them is
bounded (portdnn_b200/csrc/umma.cuh: mbar_wait), and on running out it fills an error record and
lets the kernel return.  The reference has no counterpart (its kernels never wait on one another).

The GPU test runs a test-only kernel (tests/cuda/wait_timeout.cu) that calls that same wait on a
barrier nobody arrives at, with a 2 ms limit, and checks the record, the time the wait took, and
that the context still computes afterwards."""
import ctypes
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests", "cuda"))


def test_helper_builds():
    import build_helpers
    assert os.path.exists(build_helpers.build())


@pytest.mark.gpu
def test_a_wait_nobody_answers_gives_up_and_reports():
    import numpy as np
    import torch

    import build_helpers
    import portdnn_b200 as pd
    from oracle import oracle as orc

    torch.cuda.init()
    torch.zeros(1, device="cuda")
    lib = ctypes.CDLL(build_helpers.build())
    lib.pdnn_test_wait_runs_out.argtypes = [ctypes.c_ulonglong, ctypes.POINTER(ctypes.c_uint),
                                            ctypes.POINTER(ctypes.c_ulonglong)]
    record, elapsed = (ctypes.c_uint * 4)(), ctypes.c_ulonglong(0)
    limit_ns = 2_000_000
    assert lib.pdnn_test_wait_runs_out(limit_ns, record, ctypes.byref(elapsed)) == 0
    assert record[0] == 1, list(record)          # kErrWaitTimeout
    assert record[1] == 0                        # the CTA that gave up
    assert record[2] == 0x700                    # the wait site handed to mbar_wait
    assert record[3] == 0                        # the parity it waited for; also: the flag reached the other warp
    assert limit_ns <= elapsed.value < 100 * limit_ns, elapsed.value
    # the library's own record is untouched and the context still computes correctly
    assert pd.device_error_record()[0] == 0
    rng = np.random.default_rng(0)
    p, po = pd.conv_params(2, 14, 14, 64, 64, 3, 1), orc.conv_params(2, 14, 14, 64, 64, 3, 1)
    x = torch.from_numpy(rng.standard_normal(2 * 14 * 14 * 64).astype(np.float32)).half()
    w = torch.from_numpy((rng.standard_normal(9 * 64 * 64) * 0.05).astype(np.float32)).half()
    y = pd.conv2d(pd.FORWARD, x.cuda(), w.cuda(), p, algorithm=pd.ALGO_IM2COL).float().cpu().numpy()
    ref = orc.conv2d(orc.FORWARD, x.float().numpy(), w.float().numpy(), po)
    assert np.abs(y - ref).max() <= 2e-2 * np.abs(ref).max()
