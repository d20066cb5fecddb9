"""Grouped forward convolution against the reference's known-answer vectors
(test/conv2d/forward_window*_stride*_groups*.cc, the 540 STRIDED cases in
tests/golden/grouped_conv2d_kat.npz; tolerance 10 ULP, test/conv2d/group_convolution_fixture.h):
the oracle on the CPU, the CUDA library through the C ABI on the GPU (HWCF and FHWC filters)."""
import numpy as np
import pytest

from conftest import ulp_diff


def _cases(golden):
    table, data = golden("grouped_conv2d")
    for row in table:
        window, stride, groups, n, h, w, c, feat, same, fhwc = [int(v) for v in row[:10]]
        yield (window, stride, groups, n, h, w, c, feat, bool(same), bool(fhwc), float(row[10]),
               data[int(row[11]):int(row[11]) + int(row[12])])


def test_oracle_matches_grouped_vectors(orc, golden):
    bad, count = [], 0
    for window, stride, groups, n, h, w, c, feat, same, fhwc, max_val, exp in _cases(golden):
        count += 1
        p = orc.conv_params(n, h, w, c, feat, window, stride, same, groups=groups)
        x = orc.iota(n * h * w * c, max_val)
        wt = orc.iota(window * window * (c // groups) * feat, max_val)  # [R][S][C/G][K]
        got = orc.conv2d(orc.FORWARD, x, wt, p)
        if got.size != exp.size or ulp_diff(got, exp).max(initial=0) > 10:
            bad.append((window, stride, groups, n, h, w, c, feat, same))
    assert count == 540
    assert bad == []


@pytest.mark.gpu
def test_gpu_matches_grouped_vectors(orc, golden):
    import torch

    import portdnn_b200 as pd
    bad = []
    for window, stride, groups, n, h, w, c, feat, same, fhwc, max_val, exp in _cases(golden):
        p = pd.conv_params(n, h, w, c, feat, window, stride, same, groups=groups, filter_format=2 if fhwc else 0)
        x = torch.from_numpy(orc.iota(n * h * w * c, max_val)).cuda()
        wt = orc.iota(window * window * (c // groups) * feat, max_val)
        if fhwc:  # the fixture transposes [R*S*C/G][K] to [K][R*S*C/G]
            wt = np.ascontiguousarray(wt.reshape(-1, feat).T).ravel()
        got = pd.conv2d(pd.FORWARD, x, torch.from_numpy(wt).cuda(), p, algorithm=pd.ALGO_IM2COL).cpu().numpy().ravel()
        if got.size != exp.size or ulp_diff(got, exp).max(initial=0) > 10:
            bad.append((window, stride, groups, n, h, w, c, feat, same, fhwc))
    assert bad == []
