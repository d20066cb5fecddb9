"""Extract the reference's known-answer vectors for the binary operators into one fixture.

Reads test/binaryop/binaryop_{add,sub,mul,div}.cc of a reference checkout as text: every
TYPED_TEST holds its expected output inline, the two operand shapes (params.lhs_dims /
params.rhs_dims, at most four extents each, broadcast against each other numpy-style) and the wrap
value of the ramps 1, 2, ..., max, 1, ... both operands are filled with
(test/binaryop/fixture.h:33-41, test/gen/iota_initialised_data.h:45-79).  Writes
tests/golden/binaryop_kat.npz: one object array of cases, each a dict
{op, name, lhs_dims, rhs_dims, max_input_val, exp_out}.

Usage:  python tests/golden/make_golden_binaryop.py --reference <portDNN checkout>
"""
import argparse
import os
import re

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
CASE_RE = re.compile(r"TYPED_TEST\((\w+),\s*(\w+)\)\s*\{(.*?)\n\}", re.S)
VEC_RE = re.compile(r"std::vector<DataType>\s+exp_out\s*=\s*\{(.*?)\};", re.S)
DIMS_RE = re.compile(r"params\.(lhs|rhs)_dims\s*=\s*\{(.*?)\};")
MAX_RE = re.compile(r"max_input_val\s*=\s*([\d.]+)")
OPS = ["add", "sub", "mul", "div"]


def parse(path, op):
    cases = []
    for _, name, body in CASE_RE.findall(open(path).read()):
        vec = VEC_RE.search(body)
        dims = dict(DIMS_RE.findall(body))
        mx = MAX_RE.search(body)
        if not (vec and "lhs" in dims and "rhs" in dims and mx):
            continue
        exp = np.asarray([float(t.strip().rstrip("f")) for t in vec.group(1).replace("\n", " ").split(",") if t.strip()],
                         dtype=np.float64)
        cases.append({"op": op, "name": name,
                      "lhs_dims": [int(v) for v in dims["lhs"].split(",") if v.strip()],
                      "rhs_dims": [int(v) for v in dims["rhs"].split(",") if v.strip()],
                      "max_input_val": float(mx.group(1)), "exp_out": exp})
    return cases


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    cases = []
    for op in OPS:
        got = parse(os.path.join(args.reference, "test", "binaryop", "binaryop_%s.cc" % op), op)
        print("%-4s %3d cases" % (op, len(got)))
        cases += got
    arr = np.empty(len(cases), dtype=object)
    for i, c in enumerate(cases):
        arr[i] = c
    out = os.path.join(HERE, "binaryop_kat.npz")
    np.savez_compressed(out, cases=arr)
    print("wrote %s: %d cases, %d bytes" % (out, len(cases), os.path.getsize(out)))


if __name__ == "__main__":
    main()
