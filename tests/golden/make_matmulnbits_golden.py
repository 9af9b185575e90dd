#!/usr/bin/env python3
"""Generate tests/golden/matmulnbits_goldens.json from the known-answer tests MIGraphX holds for the
weight-only int4 path: test/onnx/verify/matmulnbits_tests.cpp (inputs, packed weights, scales, packed
zero points and the expected outputs of four MatMulNBits models evaluated on `ref`).

The ONNX parser cannot be built here (no protobuf), so the test that reads this fixture rebuilds by
hand the operator sequence the parser emits (src/onnx/parse_matmulnbits.cpp:85-158) and checks the
numpy restatement, and the `ref` target's own operators, against the expected outputs.

Usage: python tests/golden/make_matmulnbits_golden.py --ref <MIGraphX source tree>
"""
import argparse
import json
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))


def _numbers(text):
    return [int(t, 16) if t.lower().startswith("0x") else float(t.rstrip("f"))
            for t in re.findall(r"0x[0-9a-fA-F]+|-?\d+\.?\d*(?:[eE][-+]?\d+)?f?", text)]


def _vector(body, name):
    m = re.search(r"std::vector<\w+>\s+" + name + r"\s*\{(.*?)\};", body, re.S)
    return _numbers(m.group(1)) if m else None


def _shape(body, name):
    m = re.search(name + r"_shape\s*=\s*migraphx::shape\{migraphx::shape::\w+,\s*\{([^}]*)\}\}", body)
    return [int(v) for v in m.group(1).split(",")] if m else None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("MIGRAPHX_SOURCE_DIR", ""))
    a = ap.parse_args()
    path = os.path.join(a.ref, "test", "onnx", "verify", "matmulnbits_tests.cpp")
    text = open(path).read()
    cases = {}
    for m in re.finditer(r"TEST_CASE\((\w+)\)\s*\{(.*?)\n\}", text, re.S):
        name, body = m.group(1), m.group(2)
        a_shape = _shape(body, "a")
        avals = _vector(body, "a")
        if avals is None or not avals:  # std::iota(a.begin(), a.end(), 0)
            n = 1
            for d in a_shape:
                n *= d
            avals = [float(i) for i in range(n)]
        out_lens = re.search(r"lens\(\)\s*==\s*std::vector<size_t>\{([^}]*)\}", body).group(1)
        cases[name] = {
            "a_shape": a_shape, "a": avals,
            "b_shape": _shape(body, "b"), "b": [int(v) for v in _vector(body, "b")],
            "scales": _vector(body, "scales"),
            "zp": [int(v) for v in _vector(body, "zp")] if _vector(body, "zp") is not None else None,
            "gold": _vector(body, "gold"), "out_lens": [int(v) for v in out_lens.split(",")],
        }
    out = os.path.join(HERE, "matmulnbits_goldens.json")
    with open(out, "w") as f:
        json.dump({"source": "test/onnx/verify/matmulnbits_tests.cpp", "cases": cases}, f, indent=1)
    print("wrote", out, sorted(cases))


if __name__ == "__main__":
    main()
