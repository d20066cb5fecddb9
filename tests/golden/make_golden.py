"""Extract the reference's own known-answer vectors into compact fixtures.

Reads the generated gtest sources of the reference checkout (conv2d,
depthwise_conv2d and pooling window/stride suites; path given by --reference)
and writes, per family, one ``.npz`` holding a case table and the concatenated
expected outputs.  Inputs are not stored: every tensor an op reads in those
tests is the ramp ``1, 2, ..., max_val, 1, 2, ...`` (reference
``test/gen/iota_initialised_data.h:45-79``), which ``golden_io.iota`` rebuilds.

The committed fixtures hold a deterministic subset (``--keep-every``) so that
they stay small; ``oracle/pin_oracle.py`` replays *all* cases straight from a
reference checkout when one is present.

Usage:  python tests/golden/make_golden.py --reference <portDNN checkout>
"""
import argparse
import os
import re

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

CASE_RE = re.compile(r"TYPED_TEST\((\w+),\s*(\w+)\)\s*\{(.*?)\n\}", re.S)
EXP_RE = re.compile(r"exp_out\s*=\s*\{(.*?)\};", re.S)
SHAPE_RE = re.compile(r"in_shape\s*=\s*\{\{(.*?)\}\}")
FEAT_RE = re.compile(r"(?:features|multiplier)\s*=\s*(\d+)")
PAD_RE = re.compile(r"PaddingMode::(SAME|VALID)")
MAXV_RE = re.compile(r"max_input_val\s*=\s*([0-9.eE+-]+)")
WS_RE = re.compile(r"(?:WindowStrideTest<\w+,\s*(\d+),\s*(\d+)>|getPoolingParams<(\d+),\s*(\d+)>)")


def _floats(txt):
    txt = txt.replace("\n", " ")
    vals = []
    for tok in txt.split(","):
        tok = tok.strip()
        if not tok:
            continue
        if tok.endswith("f"):
            tok = tok[:-1]
        vals.append(float(tok))
    return np.asarray(vals, dtype=np.float64)


def parse_file(path):
    """Yield dicts for every TYPED_TEST case in one generated test source."""
    src = open(path).read()
    m = WS_RE.search(src)
    if not m:
        return
    window = int(m.group(1) or m.group(3))
    stride = int(m.group(2) or m.group(4))
    for suite, name, body in CASE_RE.findall(src):
        e = EXP_RE.search(body)
        s = SHAPE_RE.search(body)
        p = PAD_RE.search(body)
        v = MAXV_RE.search(body)
        if not (e and s and p and v):
            continue
        f = FEAT_RE.search(body)
        yield dict(
            name=name,
            window=window,
            stride=stride,
            in_shape=[int(t) for t in s.group(1).split(",")],
            feat=int(f.group(1)) if f else 0,
            same=1 if p.group(1) == "SAME" else 0,
            max_val=float(v.group(1)),
            exp=_floats(e.group(1)),
        )


CONV_PASSES = {"forward": 0, "input_backprop": 1, "filter_backprop": 2}
POOL_OPS = {"max": 0, "maxwithnan": 1, "avg": 2}


def family_files(ref, family):
    """Return [(path, op_code, dir_or_pass_code)] for a family."""
    out = []
    if family in ("conv2d", "depthwise_conv2d"):
        d = os.path.join(ref, "test", family)
        for fn in sorted(os.listdir(d)):
            m = re.match(r"(forward|input_backprop|filter_backprop)_window(\d+)_stride(\d+)\.cc$", fn)
            if m:
                out.append((os.path.join(d, fn), 0, CONV_PASSES[m.group(1)]))
    elif family == "pooling":
        d = os.path.join(ref, "test", "pooling")
        for fn in sorted(os.listdir(d)):
            m = re.match(r"(max|maxwithnan|avg)_window(\d+)_stride(\d+)_(forward|grad)\.cc$", fn)
            if m:
                out.append((os.path.join(d, fn), POOL_OPS[m.group(1)], 0 if m.group(4) == "forward" else 1))
    return out


def collect(ref, family, keep_every=1, max_out=None):
    """Case table columns: op, pass/dir, window, stride, N, H, W, C, feat, same,
    max_val, offset, length."""
    rows, chunks, off, idx = [], [], 0, 0
    for path, op, pd in family_files(ref, family):
        for c in parse_file(path):
            idx += 1
            if keep_every > 1 and (idx % keep_every) != 0:
                continue
            if max_out is not None and c["exp"].size > max_out:
                continue
            n, h, w, ch = c["in_shape"]
            rows.append([op, pd, c["window"], c["stride"], n, h, w, ch, c["feat"], c["same"],
                         c["max_val"], off, c["exp"].size])
            chunks.append(c["exp"])
            off += c["exp"].size
    table = np.asarray(rows, dtype=np.float64)
    data = np.concatenate(chunks) if chunks else np.zeros(0)
    return table, data


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--keep-every", type=int, default=6)
    ap.add_argument("--out", default=HERE)
    args = ap.parse_args()
    for fam in ("conv2d", "depthwise_conv2d", "pooling"):
        table, data = collect(args.reference, fam, args.keep_every)
        # every expected value of these suites is exactly representable in fp32
        d32 = data.astype(np.float32)
        path = os.path.join(args.out, fam + "_kat.npz")
        np.savez_compressed(path, table=table, data=d32)
        print(fam, "cases", table.shape[0], "values", data.size, "bytes", os.path.getsize(path))


if __name__ == "__main__":
    main()
