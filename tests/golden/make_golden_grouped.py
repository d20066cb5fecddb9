"""Extract the reference's known-answer vectors of grouped forward convolution
(test/conv2d/forward_window*_stride*_groups*.cc) into tests/golden/grouped_conv2d_kat.npz.

Both group formats are kept: STRIDED (channels and features of a group are contiguous) and INTERLEAVED
(the group is the fastest index of both axes; HWCF filters only).  The expected values are in the order
the library writes them; the fixture (test/conv2d/group_convolution_fixture.h:41-77) reorders the iota
input and filter for the INTERLEAVED cases, and the replaying tests do the same.
Case table columns: window, stride, groups, N, H, W, C, features, same, fhwc, max_val, offset, length,
interleaved.

Usage:  python tests/golden/make_golden_grouped.py --reference <portDNN checkout>
"""
import argparse
import os
import re

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
CASE_RE = re.compile(r"TYPED_TEST\((\w+),\s*(\w+)\)\s*\{(.*?)\n\}", re.S)


def _floats(txt):
    return np.asarray([float(t.strip().rstrip("f")) for t in txt.replace("\n", " ").split(",") if t.strip()])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    d = os.path.join(args.reference, "test", "conv2d")
    rows, chunks, off = [], [], 0
    for fn in sorted(os.listdir(d)):
        m = re.match(r"forward_window(\d+)_stride(\d+)_groups(\d+)\.cc$", fn)
        if not m:
            continue
        window, stride, groups = (int(v) for v in m.groups())
        for _, name, body in CASE_RE.findall(open(os.path.join(d, fn)).read()):
            interleaved = 1 if "BatchFormat::INTERLEAVED" in body else 0
            exp = _floats(re.search(r"exp_out\s*=\s*\{(.*?)\};", body, re.S).group(1))
            n, h, w, c = (int(v) for v in re.search(r"in_shape\s*=\s*\{\{(.*?)\}\}", body).group(1).split(","))
            feat = int(re.search(r"features\s*=\s*(\d+)", body).group(1))
            same = 1 if "PaddingMode::SAME" in body else 0
            fhwc = 1 if "FilterFormat::FHWC" in body else 0
            max_val = float(re.search(r"max_input_val\s*=\s*([0-9.eE+-]+)", body).group(1))
            rows.append([window, stride, groups, n, h, w, c, feat, same, fhwc, max_val, off, exp.size, interleaved])
            chunks.append(exp)
            off += exp.size
    table = np.asarray(rows, dtype=np.float64)
    data = np.concatenate(chunks).astype(np.float32)
    path = os.path.join(HERE, "grouped_conv2d_kat.npz")
    np.savez_compressed(path, table=table, data=data)
    print("grouped conv2d cases", table.shape[0], "values", data.size, "bytes", os.path.getsize(path))


if __name__ == "__main__":
    main()
