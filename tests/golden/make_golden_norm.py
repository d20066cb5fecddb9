"""Extract the reference's known-answer vectors for softmax and batchnorm into one fixture.

Reads test/softmax/softmax_{forward,grad}.cc and test/batchnorm/batchnorm_{forward,gradient}_
{frozen,training}.cc of a reference checkout as text: every TYPED_TEST holds its expected vectors
inline, the input shape, and the wrap value of the ramps 1, 2, ..., max, 1, ... the fixture feeds
the operator with (test/gen/iota_initialised_data.h:45-79).  Writes tests/golden/norm_kat.npz:
one object array of cases, each a dict {op, shape, scalars..., vectors...}.

Usage:  python tests/golden/make_golden_norm.py --reference <portDNN checkout>
"""
import argparse
import os
import re

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
CASE_RE = re.compile(r"TYPED_TEST\((\w+),\s*(\w+)\)\s*\{(.*?)\n\}", re.S)
VEC_RE = re.compile(r"std::vector<DataType>\s+(\w+)\s*=\s*\{(.*?)\};", re.S)
SHAPE_RE = re.compile(r"in_shape\s*=\s*\{\{(.*?)\}\}")
SCALAR_RE = re.compile(r"const\s+(?:DataType|float|bool)\s+(\w+)\s*=\s*([\w.+-]+);")

FILES = {
    "softmax_forward": "test/softmax/softmax_forward.cc",
    "softmax_grad": "test/softmax/softmax_grad.cc",
    "batchnorm_forward_frozen": "test/batchnorm/batchnorm_forward_frozen.cc",
    "batchnorm_forward_training": "test/batchnorm/batchnorm_forward_training.cc",
    "batchnorm_gradient_frozen": "test/batchnorm/batchnorm_gradient_frozen.cc",
    "batchnorm_gradient_training": "test/batchnorm/batchnorm_gradient_training.cc",
}


def _floats(txt):
    return np.asarray([float(t.strip().rstrip("f")) for t in txt.replace("\n", " ").split(",") if t.strip()],
                      dtype=np.float64)


def parse(path, op):
    cases = []
    for _, name, body in CASE_RE.findall(open(path).read()):
        shape = SHAPE_RE.search(body)
        if not shape:
            continue
        case = {"op": op, "name": name, "shape": [int(v) for v in shape.group(1).split(",")]}
        for vname, vals in VEC_RE.findall(body):
            case[vname] = _floats(vals)
        for sname, val in SCALAR_RE.findall(body):
            case[sname] = {"true": 1.0, "false": 0.0}.get(val, None) if val in ("true", "false") else float(val)
        cases.append(case)
    return cases


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    cases = []
    for op, rel in FILES.items():
        got = parse(os.path.join(args.reference, rel), op)
        print("%-28s %3d cases" % (op, len(got)))
        cases += got
    np.savez_compressed(os.path.join(HERE, "norm_kat.npz"), cases=np.array(cases, dtype=object))


if __name__ == "__main__":
    main()
