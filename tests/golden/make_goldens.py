#!/usr/bin/env python3
"""Extract the reference's own golden vectors for the quantized-matmul path.

Reads the `const NAME: [T; N] = [...]` / `const NAME: &[T] = &[...]` tables out
of the reference's Rust test modules (as text; nothing is compiled or run) and
writes them to `frink_goldens.json` beside this script.  The tables are test
DATA (bytes llama.cpp's encoders produced, values an independent dequantizer
produced); the oracle under `oracle/` is pinned against them.

Usage: python tests/golden/make_goldens.py [path-to-frink-checkout]
"""
import json
import os
import re
import sys

WANTED = {
    "crates/frink-quant/src/encode.rs": [
        "LLAMA_CPP_Q8_0_GOLDEN", "TIE_BLOCK_F16_BITS", "LLAMA_CPP_TIE_BLOCK_GOLDEN",
    ],
    "crates/frink-quant/src/encode/testdata.rs": ["REAL_WEIGHT_BLOCKS"],
    "crates/frink-quant/src/encode/q4_k.rs": ["LLAMA_CPP_Q4_K_GOLDEN"],
    "crates/frink-quant/src/encode/q5_k.rs": ["LLAMA_CPP_Q5_K_GOLDEN"],
    "crates/frink-quant/src/encode/q6_k.rs": ["LLAMA_CPP_Q6_K_GOLDEN"],
    "crates/frink-quant/src/lib.rs": [
        "Q4_K_TEST_BLOCK", "Q4_K_GOLDEN", "Q5_K_TEST_BLOCK", "Q5_K_GOLDEN", "Q6_K_TEST_BLOCK", "Q6_K_GOLDEN",
        "Q6_K_SIGNED_SCALES_TEST_BLOCK", "Q6_K_SIGNED_SCALES_GOLDEN",
        "Q6_K_SIGNED_TEST_BLOCK", "Q6_K_SIGNED_GOLDEN",
        "MXFP4_GGUF_TEST_BLOCKS", "MXFP4_GGUF_GOLDEN",
    ],
}


def parse_literal(tok):
    tok = tok.strip().replace("_", "")
    for suffix in ("u8", "u16", "u32", "i8", "i16", "i32", "f32", "f64"):
        if tok.endswith(suffix) and not tok.startswith("0x"):
            tok = tok[: -len(suffix)]
    if tok.lower().startswith("0x") or tok.lower().startswith("-0x"):
        return int(tok, 16)
    if re.fullmatch(r"-?\d+", tok):
        return int(tok)
    return float(tok)


def extract(text, name):
    m = re.search(r"const\s+" + re.escape(name) + r"\s*:\s*[^=]+=\s*&?\[", text)
    if not m:
        raise KeyError(name)
    i = m.end()
    depth = 1
    j = i
    while depth:
        c = text[j]
        depth += c == "["
        depth -= c == "]"
        j += 1
    body = re.sub(r"//[^\n]*", "", text[i : j - 1])
    return [parse_literal(t) for t in body.split(",") if t.strip()]


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_goldens.py <checkout of antonellof/frink>")
    root = sys.argv[1]
    out = {"source": "antonellof/frink v0.63.0", "tables": {}}
    for rel, names in WANTED.items():
        text = open(os.path.join(root, rel)).read()
        for name in names:
            out["tables"][name] = {"file": rel, "values": extract(text, name)}
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "frink_goldens.json")
    with open(dst, "w") as f:
        json.dump(out, f, separators=(",", ":"))
    for k, v in out["tables"].items():
        print(f"{k}: {len(v['values'])} values from {v['file']}")


if __name__ == "__main__":
    main()
