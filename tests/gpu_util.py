"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

import portdnn_b200 as pd

TORCH_DTYPES = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
# Parity bars: relative error (max |diff| / max |ref|) against the oracle on the same rounded inputs.
TOL = {"f32": 1e-4, "f16": 2e-2, "bf16": 2e-2}


def to_dev(a, dtype):
    """numpy float32 -> CUDA tensor of the given dtype (rounded once)."""
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to("cuda").to(TORCH_DTYPES[dtype]).contiguous()


def rounded(a, dtype):
    """What the device sees: the float32 values after one rounding to dtype."""
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(TORCH_DTYPES[dtype]).float().numpy()


def to_host(t):
    return t.detach().float().cpu().numpy().ravel()


def assert_no_device_error():
    rec = pd.device_error_record()
    assert rec[0] == 0, "tensor-core kernel reported %s" % rec
