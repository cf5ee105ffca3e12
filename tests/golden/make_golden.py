#!/usr/bin/env python3
"""Extracts the reference's own known-answer vectors for the quantized-matmul path into JSON fixtures.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

It reads the reference's test sources as text (nothing is executed) and writes, next to this script:

  mxfp4_kat.json       packed words, e8m0 scales and the 128 expected fp32 values of MXFP4ReferenceTests
                       (Tests/IngotTests/KernelCaseMXFP4.swift:141-158; produced there by mlx's mx.dequantize)
  swiglu_oai_kat.json  the 13x9 grid of SwigluOAIReferenceTests (Tests/IngotTests/KernelCaseGptOss.swift:68-85;
                       produced there by mlx-lm's swiglu_oai)
  router_vectors.json  the seven router cases of ref/router_vectors.json (mlx-lm 0.32.2 router modules on random
                       logits with exact k-th place ties in rows 0-1)
  format_kat.json      the nibble-order and affine dequantisation known answers of
                       Tests/IngotTests/FormatTests.swift:39-70 (inputs as the test builds them; the expected values
                       are evaluated here with scalar Python floats, independently of the oracle)

The fixtures are data, not code; the tests under tests/ compare the oracle (and, on a GPU, the kernels) with them.
"""
import json
import os
import re
import struct
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def swift_array(text: str, name: str) -> str:
    m = re.search(r"static let " + re.escape(name) + r"\s*:\s*\[[A-Za-z0-9]+\]\s*=\s*\[(.*?)\]", text, re.S)
    if not m:
        raise SystemExit(f"array {name} not found")
    return m.group(1)


def floats(body: str):
    return [float(v) for v in re.findall(r"-?\d+(?:\.\d+)?(?:e-?\d+)?", body)]


def f32_bits(v: float) -> int:
    return struct.unpack("<I", struct.pack("<f", v))[0]


def bf16_round(v: float) -> float:
    u = f32_bits(v)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return struct.unpack("<f", struct.pack("<I", u & 0xFFFFFFFF))[0]


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <checkout of the reference>")
    ref = sys.argv[1]
    tests = os.path.join(ref, "Tests", "IngotTests")

    # --- MXFP4 ---------------------------------------------------------------------------------------------
    t = open(os.path.join(tests, "KernelCaseMXFP4.swift"), encoding="utf-8").read()
    t = t[t.index("struct MXFP4ReferenceTests"):]
    words = [int(v.replace("_", ""), 16) for v in re.findall(r"0x[0-9A-Fa-f_]+", swift_array(t, "words"))]
    scales = [int(v) for v in re.findall(r"\d+", swift_array(t, "scales"))]
    values = floats(swift_array(t, "values"))
    assert len(words) == 16 and len(scales) == 4 and len(values) == 128
    json.dump(
        {"source": "Tests/IngotTests/KernelCaseMXFP4.swift:141-158", "rows": 2, "cols": 64, "words": words,
         "scales": scales, "values": values, "value_bits": [f32_bits(v) for v in values],
         "e2m1": [0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6]},
        open(os.path.join(HERE, "mxfp4_kat.json"), "w"))

    # --- swiglu_oai ----------------------------------------------------------------------------------------
    t = open(os.path.join(tests, "KernelCaseGptOss.swift"), encoding="utf-8").read()
    t = t[t.index("struct SwigluOAIReferenceTests"):]
    g, u, y = floats(swift_array(t, "g")), floats(swift_array(t, "u")), floats(swift_array(t, "y"))
    assert len(y) == len(g) * len(u) == 117
    json.dump({"source": "Tests/IngotTests/KernelCaseGptOss.swift:68-85", "limit": 7.0, "g": g, "u": u, "y": y,
               "tol": 1e-6}, open(os.path.join(HERE, "swiglu_oai_kat.json"), "w"))

    # --- router --------------------------------------------------------------------------------------------
    rv = json.load(open(os.path.join(ref, "ref", "router_vectors.json")))
    assert len(rv["cases"]) == 7
    json.dump({"source": "ref/router_vectors.json; " + rv["source"], "cases": rv["cases"]},
              open(os.path.join(HERE, "router_vectors.json"), "w"))

    # --- format --------------------------------------------------------------------------------------------
    N, K = 2, 128
    q = [(i * 7 + 3) % 16 for i in range(N * K)]
    s = [0.5, 0.25, 1.0, 2.0]
    b = [-1.0, 0.0, 0.5, 3.0]
    expected = []
    for r in range(N):
        for j in range(K):
            gi = r * 2 + j // 64
            expected.append(bf16_round(s[gi]) * float(q[r * K + j]) + bf16_round(b[gi]))
    json.dump(
        {"source": "Tests/IngotTests/FormatTests.swift:39-70", "pack4_in": [1, 2, 3, 4, 5, 6, 7, 8],
         "pack4_out": [0x87654321], "N": N, "K": K, "codes": q, "scales": s, "biases": b, "expected": expected},
        open(os.path.join(HERE, "format_kat.json"), "w"))
    print("wrote mxfp4_kat.json swiglu_oai_kat.json router_vectors.json format_kat.json")


if __name__ == "__main__":
    main()
