"""Extract the reference's remaining known-answer tests for the convolution path into fixtures.

Covers the suites that tests/golden/make_golden.py (the generated window/stride families) does
not: the matmul suites (test/matmul/matmul_batch*_beta*_*.cc, matmul_offset.cc), the hand-written
convolution tests (test/conv2d/{forward,input_backprop,filter_backprop}_1x1.cc,
simple_convolution.cc, convolution_offsets.cc), pointwise forward / gradient
(test/pointwise/*_{forward,grad}.cc), bias add (test/bias/test_bias.cc), max pooling with NaNs
(test/pooling/max_pooling_with_nan.cc) and pooling with pointer offsets (test/pooling/pooling_offset.cc).

Every case is stored with what the fixture feeds the operator (sizes, ramp maximum, offsets,
literal inputs where the test spells them out) and the expected output; inputs that are ramps are
rebuilt at test time (test/gen/iota_initialised_data.h:45-97).

Usage:  python tests/golden/make_golden_misc.py --reference <portDNN checkout>
Writes tests/golden/matmul_kat.npz and tests/golden/misc_kat.json.
"""
import argparse
import glob
import json
import math
import os
import re

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
CASE_RE = re.compile(r"TYPED_TEST\((\w+),\s*(\w+)\)\s*\{(.*?)\n\}", re.S)


def floats(txt):
    out = []
    for tok in txt.replace("\n", " ").split(","):
        tok = tok.strip()
        if not tok:
            continue
        if tok in ("nan", "-nan"):
            out.append(float("nan"))
        elif tok == "min":
            out.append(-3.4028234663852886e38)
        else:
            out.append(float(tok.rstrip("f")))
    return out


def vectors(body):
    """All std::vector<DataType> definitions of a test body: name -> list (braced lists and
    `name(count, value)` fills)."""
    found = {}
    for name, txt in re.findall(r"std::vector<DataType>\s+(\w+)\s*=\s*\{(.*?)\};", body, re.S):
        found[name] = floats(txt)
    for name, count, val in re.findall(r"std::vector<DataType>\s+(\w+)\((\d+),\s*(\w+)\);", body):
        found[name] = floats(val) * int(count)
    return found


def jsonable(v):
    return [None if isinstance(x, float) and math.isnan(x) else x for x in v]


# ---- matmul -----------------------------------------------------------------------------------
def matmul_cases(ref):
    cases = []
    for path in sorted(glob.glob(os.path.join(ref, "test", "matmul", "matmul_batch*_beta*_*.cc"))) + \
            [os.path.join(ref, "test", "matmul", "matmul_offset.cc")]:
        src = open(path).read()
        fixtures2 = {m[0]: (m[1], m[2]) for m in re.findall(r"using (\w+) =\s*MatmulFixture<\w+,\s*(\w+),\s*(\w+)>", src)}
        for suite, name, body in CASE_RE.findall(src):
            exp = vectors(body).get("exp_out") or vectors(body).get("exp")
            ints = {k: int(v) for k, v in re.findall(r"const int (\w+) = (\d+);", body)}
            beta = re.search(r"beta = static_cast<DataType>\(([0-9.]+)\)", body)
            run = re.search(r"this->run\((.*?)\);", body, re.S).group(1).split(",")
            offs = [a.strip() for a in run[6:9]]
            offs = [ints.get(a, int(a) if a.isdigit() else 0) for a in offs]
            maxv = re.search(r"max_input_val = ([0-9.]+)", body)
            tl, tr = fixtures2[suite]
            cases.append(dict(name=suite + "." + name, tl=tl == "true", tr=tr == "true", batches=ints["batches"], m=ints["m"],
                              k=ints["k"], n=ints["n"], beta=float(beta.group(1)) if beta else 0.0, offsets=offs,
                              max_val=float(maxv.group(1)) if maxv else 0.0, exp=exp))
    return cases


# ---- hand-written convolution tests ---------------------------------------------------------------
FIELDS = ["channels", "features", "batch", "in_rows", "in_cols", "window_rows", "window_cols", "stride_rows", "stride_cols",
          "out_rows", "out_cols", "pad_rows", "pad_cols", "dilation_rows", "dilation_cols"]


def param_helpers(src):
    """The file's `Conv2DParams get_xxx(int a, ...)` helpers as Python callables returning a dict."""
    helpers = {}
    for name, args, body in re.findall(r"Conv2DParams (get_\w+)\((.*?)\)\s*\{(.*?)\n\}", src, re.S):
        argn = [a.split()[-1] for a in args.split(",") if a.strip()]

        def make(argn=argn, body=body):
            def fn(*vals):
                env = dict(zip(argn, vals))
                base = re.search(r"auto params = (get_\w+)\((.*?)\);", body)
                p = helpers[base.group(1)](*[eval(a, {}, env) for a in base.group(2).split(",") if a.strip()]) if base else {}
                for f, expr in re.findall(r"params\.(\w+) = (.*?);", body):
                    p[f] = int(eval(expr.replace("/", "//"), {}, env))
                return p
            return fn
        helpers[name] = make()
    return helpers


def same_padding(p):
    """helpers::add_padding_to(params, SAME), include/portdnn/helpers/padding.h:46-88."""
    for d in ("rows", "cols"):
        inp, win, st = p["in_" + d], p["window_" + d], p["stride_" + d]
        out = -(-inp // st)
        need = max((out - 1) * st + win - inp, 0)
        p["out_" + d], p["pad_" + d] = out, need // 2
    return p


def conv_cases(ref):
    cases = []
    for fname in ("forward_1x1.cc", "input_backprop_1x1.cc", "filter_backprop_1x1.cc", "simple_convolution.cc",
                  "convolution_offsets.cc"):
        src = open(os.path.join(ref, "test", "conv2d", fname)).read()
        helpers = param_helpers(src)
        for suite, name, body in CASE_RE.findall(src):
            vecs = vectors(body)
            exp = vecs.get("exp") or vecs.get("exp_out")
            call = re.search(r"params = (get_\w+)\((.*?)\);", body)
            p = helpers[call.group(1)](*[int(a) for a in call.group(2).split(",") if a.strip()])
            for f, expr in re.findall(r"params\.(\w+) = (\d+);", body):
                p[f] = int(expr)
            if "add_padding_to" in body:
                p = same_padding(p)
            conv_type = re.search(r"conv_type::(\w+)", body).group(1)
            args = re.search(r"test_conv<.*?>\(\s*(.*?)\);", body, re.S).group(1).replace("\n", " ").split(",")
            extra = [a.strip() for a in args[2:]]
            maxv = 0.0
            if extra:
                m = re.search(r"max_input_val = ([0-9.]+)", body)
                maxv = float(m.group(1)) if extra[0] == "max_input_val" and m else float(extra[0])
            offs = [int(a) for a in extra[1:4]] + [0] * (3 - len(extra[1:4]))
            cases.append(dict(name="%s.%s.%s" % (fname[:-3], suite, name), params=[p[f] for f in FIELDS],
                              conv_type={"Forward": 0, "InputBackprop": 1, "FilterBackprop": 2}[conv_type], max_val=maxv,
                              offsets=offs, exp=exp))
    return cases


# ---- pointwise, bias, pooling -----------------------------------------------------------------------
def pointwise_cases(ref):
    ops = {"relu": 0, "tanh": 1, "exp": 3, "log": 4, "floor": 5, "sqrt": 6}
    cases = []
    for path in sorted(glob.glob(os.path.join(ref, "test", "pointwise", "*_forward.cc")) +
                       glob.glob(os.path.join(ref, "test", "pointwise", "*_grad.cc"))):
        base = os.path.basename(path)[:-3]
        op, direction = base.rsplit("_", 1)
        for suite, name, body in CASE_RE.findall(open(path).read()):
            signed = re.search(r"iota_initialised_signed_data<DataType>\((\d+)\)", body)
            plain = re.search(r"iota_initialised_data<DataType>\((\d+),", body) or re.search(r"iota_initialised_data\((\d+),", body)
            vecs = vectors(body)
            if "exp_out" not in vecs or not (signed or plain or "input" in vecs):
                continue
            cases.append(dict(name=base + "." + name, op=ops[op], grad=direction == "grad",
                              signed_n=int(signed.group(1)) if signed else 0, plain_n=int(plain.group(1)) if plain and not signed else 0,
                              input=jsonable(vecs["input"]) if "input" in vecs else None, exp=jsonable(vecs["exp_out"])))
    return cases


def bias_cases(ref):
    cases = []
    for suite, name, body in CASE_RE.findall(open(os.path.join(ref, "test", "bias", "test_bias.cc")).read()):
        shape = [int(t) for t in re.search(r"in_shape = \{\{(.*?)\}\}", body).group(1).split(",")]
        maxv = float(re.search(r"max_input_val = ([0-9.]+)", body).group(1))
        cases.append(dict(name=name, shape=shape, max_val=maxv, exp=vectors(body)["exp_out"]))
    return cases


def pooling_cases(ref):
    cases = []
    src = open(os.path.join(ref, "test", "pooling", "max_pooling_with_nan.cc")).read()
    for suite, name, body in CASE_RE.findall(src):
        vecs = vectors(body)
        shape = [int(t) for t in re.search(r"in_shape = \{\{(.*?)\}\}", body).group(1).split(",")]
        win, st = [int(v) for v in re.search(r"getPoolingParams<(\d+),\s*(\d+)>", body).groups()]
        same = "PaddingMode::SAME" in body
        op = 1 if "pooling::MaxWithNan" in body else 0
        if "test_forward" in body:
            cases.append(dict(name="nan." + name, kind="forward", op=op, shape=shape, window=win, stride=st, same=same,
                              input=jsonable(vecs["input"]), exp=jsonable(vecs["exp_out"])))
        else:
            cases.append(dict(name="nan." + name, kind="max_grad", op=op, shape=shape, window=win, stride=st, same=same,
                              input=jsonable(vecs["input_data"]), errors=jsonable(vecs["input_errors"]),
                              exp=jsonable(vecs["exp_out"])))
    src = open(os.path.join(ref, "test", "pooling", "pooling_offset.cc")).read()
    kinds = {"PoolingOffsetAvgForward": ("forward", 2), "PoolingOffsetMaxForward": ("forward", 0),
             "PoolingOffsetAvgBackprop": ("avg_grad", 2), "PoolingOffsetMaxBackprop": ("max_grad", 0)}
    for suite, name, body in CASE_RE.findall(src):
        shape = [int(t) for t in re.search(r"in_shape = \{+(.*?)\}+", body).group(1).split(",")]
        win, st = [int(v) for v in re.search(r"getPoolingParams<(\d+),\s*(\d+)>", body).groups()]
        args = [a.strip() for a in re.search(r"test_pool\((.*?)\);", body, re.S).group(1).split(",")]
        if suite not in kinds:
            continue
        kind, op = kinds[suite]
        maxv = re.search(r"max_input_val = ([0-9.]+)", body)
        vecs = vectors(body)
        cases.append(dict(name="offset.%s.%s" % (suite, name), kind=kind, op=op, shape=shape, window=win, stride=st,
                          same="PaddingMode::SAME" in body, max_val=float(maxv.group(1)) if maxv else float(args[2]),
                          offsets=[int(a) for a in args[3:]], exp=vecs.get("exp_out") or vecs.get("exp")))
    return cases


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    mm = matmul_cases(args.reference)
    table = np.asarray([[c["tl"], c["tr"], c["batches"], c["m"], c["k"], c["n"], c["beta"], c["max_val"]] + c["offsets"] +
                        [len(c["exp"])] for c in mm], dtype=np.float64)
    np.savez_compressed(os.path.join(HERE, "matmul_kat.npz"), table=table,
                        data=np.concatenate([np.asarray(c["exp"], dtype=np.float64) for c in mm]),
                        names=np.asarray([c["name"] for c in mm]))
    misc = dict(conv2d=conv_cases(args.reference), pointwise=pointwise_cases(args.reference), bias=bias_cases(args.reference),
                pooling=pooling_cases(args.reference))
    with open(os.path.join(HERE, "misc_kat.json"), "w") as f:
        json.dump(misc, f, separators=(",", ":"))
    print("matmul %d cases; conv2d %d, pointwise %d, bias %d, pooling %d" %
          (len(mm), len(misc["conv2d"]), len(misc["pointwise"]), len(misc["bias"]), len(misc["pooling"])))


if __name__ == "__main__":
    main()
