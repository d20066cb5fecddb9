"""Grouped forward convolution against the reference's known-answer vectors
(test/conv2d/forward_window*_stride*_groups*.cc: 540 STRIDED and 360 INTERLEAVED cases in
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
               data[int(row[11]):int(row[11]) + int(row[12])], int(row[13]))


def _operands(orc, window, groups, n, h, w, c, feat, fhwc, interleaved, max_val):
    """Input and filter as the fixture hands them to the library (group_convolution_fixture.h:41-77):
    iota data; INTERLEAVED moves the group index behind the channel (feature) index; FHWC moves the
    feature axis to the front."""
    x = orc.iota(n * h * w * c, max_val)
    wt = orc.iota(window * window * (c // groups) * feat, max_val)  # [R][S][C/G][K]
    if interleaved:
        x = np.ascontiguousarray(x.reshape(-1, groups, c // groups).transpose(0, 2, 1)).ravel()
        wt = np.ascontiguousarray(wt.reshape(-1, groups, feat // groups).transpose(0, 2, 1)).ravel()
    if fhwc:
        wt = np.ascontiguousarray(wt.reshape(-1, feat).T).ravel()
    return x, wt


def test_oracle_matches_grouped_vectors(orc, golden):
    bad, count = [], [0, 0]
    for window, stride, groups, n, h, w, c, feat, same, fhwc, max_val, exp, interleaved in _cases(golden):
        count[interleaved] += 1
        p = orc.conv_params(n, h, w, c, feat, window, stride, same, groups=groups, group_format=interleaved)
        x, wt = _operands(orc, window, groups, n, h, w, c, feat, False, interleaved, max_val)  # the oracle reads HWCF
        got = orc.conv2d(orc.FORWARD, x, wt, p)
        if got.size != exp.size or ulp_diff(got, exp).max(initial=0) > 10:
            bad.append((window, stride, groups, n, h, w, c, feat, same, interleaved))
    assert count == [540, 360]
    assert bad == []


@pytest.mark.gpu
def test_gpu_matches_grouped_vectors(orc, golden):
    import torch

    import portdnn_b200 as pd
    bad = []
    for window, stride, groups, n, h, w, c, feat, same, fhwc, max_val, exp, interleaved in _cases(golden):
        p = pd.conv_params(n, h, w, c, feat, window, stride, same, groups=groups, filter_format=2 if fhwc else 0,
                           group_format=interleaved)
        x, wt = _operands(orc, window, groups, n, h, w, c, feat, fhwc, interleaved, max_val)
        got = pd.conv2d(pd.FORWARD, torch.from_numpy(x).cuda(), torch.from_numpy(wt).cuda(), p,
                        algorithm=pd.ALGO_IM2COL).cpu().numpy().ravel()
        if got.size != exp.size or ulp_diff(got, exp).max(initial=0) > 10:
            bad.append((window, stride, groups, n, h, w, c, feat, same, fhwc, interleaved))
    assert bad == []
