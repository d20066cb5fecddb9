"""Pin the CPU oracle against the reference's own known-answer vectors.

With --reference <portDNN checkout> every generated conv2d / depthwise_conv2d / pooling
case of the reference's test suite is replayed (about 25 000 cases); without it the
committed subset under tests/golden/ is replayed.  Tolerances are the reference's own:
10 ULP for conv and depthwise (test/conv2d/convolution_fixture.h:152), exact for max
pooling and its gradient, 8 ULP for average pooling (test/pooling/pooling_fixture.h:107-134,
212-215).

Usage:  python oracle/pin_oracle.py [--reference <checkout>]
"""
import argparse
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

from oracle import oracle as orc  # noqa: E402


def ulp_diff(a, b):
    a = np.asarray(a, dtype=np.float32)
    b = np.asarray(b, dtype=np.float32)
    ia = a.view(np.int32).astype(np.int64)
    ib = b.view(np.int32).astype(np.int64)
    ia = np.where(ia < 0, -(ia & 0x7FFFFFFF), ia)
    ib = np.where(ib < 0, -(ib & 0x7FFFFFFF), ib)
    return np.abs(ia - ib)


def run_case(family, row, exp):
    op, pd, window, stride, n, h, w, c, feat, same, max_val = [int(v) for v in row[:10]] + [float(row[10])]
    if family == "conv2d":
        p = orc.conv_params(n, h, w, c, feat, window, stride, bool(same))
        n_in, n_fil, _ = orc.conv_sizes(pd, p)
        got = orc.conv2d(pd, orc.iota(n_in, max_val), orc.iota(n_fil, max_val), p)
        tol = 10
    elif family == "depthwise_conv2d":
        p = orc.depthwise_params(n, h, w, c, feat, window, stride, bool(same))
        n_in, n_fil, _ = orc.depthwise_sizes(pd, p)
        got = orc.depthwise_conv2d(pd, orc.iota(n_in, max_val), orc.iota(n_fil, max_val), p)
        tol = 10
    else:
        p = orc.pool_params(n, h, w, c, window, stride, bool(same))
        x = orc.iota(n * h * w * c, max_val)
        if pd == 0:
            got = orc.pool_forward(op, x, p)
            tol = 8 if op == orc.POOL_AVERAGE else 0
        elif op == orc.POOL_AVERAGE:
            got = orc.pool_avg_grad(orc.iota(n * p.out_rows * p.out_cols * c, max_val), p)
            tol = 8
        else:
            # the reference fixture always runs the plain Max forward first
            # (test/pooling/pooling_fixture.h:172-176)
            y = orc.pool_forward(orc.POOL_MAX, x, p)
            got = orc.pool_max_grad(op, x, y, orc.iota(y.size, max_val), p)
            tol = 0
    if got.size != exp.size:
        return False, "size %d != %d" % (got.size, exp.size)
    d = ulp_diff(got, exp.astype(np.float32))
    return bool(d.max(initial=0) <= tol), "max ulp %d" % d.max(initial=0)


def replay(family, table, data):
    bad = 0
    for row in table:
        off, ln = int(row[11]), int(row[12])
        ok, msg = run_case(family, row, data[off:off + ln])
        if not ok:
            bad += 1
            if bad <= 5:
                print("  MISMATCH", family, row[:11].tolist(), msg)
    return table.shape[0], bad


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None)
    args = ap.parse_args()
    total_bad = 0
    for fam in ("conv2d", "depthwise_conv2d", "pooling"):
        if args.reference:
            sys.path.insert(0, os.path.join(os.path.dirname(HERE), "tests", "golden"))
            import make_golden
            table, data = make_golden.collect(args.reference, fam, 1)
        else:
            z = np.load(os.path.join(os.path.dirname(HERE), "tests", "golden", fam + "_kat.npz"))
            table, data = z["table"], z["data"]
        n, bad = replay(fam, table, data)
        total_bad += bad
        print("%-18s %6d cases, %d mismatches" % (fam, n, bad))
    sys.exit(1 if total_bad else 0)


if __name__ == "__main__":
    main()
