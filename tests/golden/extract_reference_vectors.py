#!/usr/bin/env python3
"""Pull the numeric literals out of the reference's in-module unit tests.

The reference (ingim/sage) keeps its known-answer vectors as `Tensor::new([...])`
literals inside `#[cfg(test)]` modules (src/ops/{map,core,reduce,gemm,conv,nn}.rs).
This script reads those Rust sources as text, finds every `fn test_*` body, and
records each `let <name> = Tensor::new(<nested literal>)` it contains, in source
order, as plain nested lists.  Only numbers are taken; what each vector means
(which op maps which input to which expected output) is restated by hand in
tests/test_oracle_golden.py, citing the reference test it follows.

Usage:  python tests/golden/extract_reference_vectors.py /path/to/reference
Writes: tests/golden/reference_vectors.json
"""
import ast
import json
import os
import re
import sys

FILES = [
    "src/ops/map.rs",
    "src/ops/core.rs",
    "src/ops/reduce.rs",
    "src/ops/gemm.rs",
    "src/ops/conv.rs",
    "src/ops/nn.rs",
]

TEST_RE = re.compile(r"fn\s+(test_[a-z0-9_]+)\s*\(\s*\)\s*\{")
LET_RE = re.compile(r"let\s+(?:mut\s+)?([a-z_0-9]+)\s*=\s*Tensor::new\s*\(")


def strip_comments(src):
    out = []
    for line in src.splitlines():
        s = line.lstrip()
        if s.startswith("//"):
            out.append("")
        else:
            out.append(line)
    return "\n".join(out)


def balanced(src, start, open_ch, close_ch):
    """Index one past the bracket that closes the one at `start`."""
    depth = 0
    i = start
    while i < len(src):
        c = src[i]
        if c == open_ch:
            depth += 1
        elif c == close_ch:
            depth -= 1
            if depth == 0:
                return i + 1
        i += 1
    raise ValueError("unbalanced")


def to_python_literal(text):
    # Rust float literals such as `1.` or `2.2621e+00` are valid Python as they are;
    # typed suffixes (1.0_f32, 3u32) are stripped.
    text = re.sub(r"_?(f32|f64|u32|i32|usize)\b", "", text)
    return ast.literal_eval(text.strip())


def extract(ref_root):
    result = {}
    for rel in FILES:
        src = strip_comments(open(os.path.join(ref_root, rel)).read())
        module = os.path.splitext(os.path.basename(rel))[0]
        tests = list(TEST_RE.finditer(src))
        for m in tests:
            body_start = src.index("{", m.end() - 1)
            body_end = balanced(src, body_start, "{", "}")
            body = src[body_start:body_end]
            vectors = []
            for lm in LET_RE.finditer(body):
                paren = lm.end() - 1
                end = balanced(body, paren, "(", ")")
                lit = body[paren + 1:end - 1]
                try:
                    value = to_python_literal(lit)
                except Exception:
                    continue
                vectors.append({"name": lm.group(1), "value": value})
            if vectors:
                line = src.count("\n", 0, m.start()) + 1
                result[f"{module}.{m.group(1)}"] = {
                    "source": f"{rel}:{line}",
                    "vectors": vectors,
                }
    return result


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: extract_reference_vectors.py <path to a checkout of ingim/sage>")
    ref_root = sys.argv[1]
    data = extract(ref_root)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.json")
    with open(out, "w") as f:
        json.dump(data, f, separators=(",", ":"))
    for k, v in data.items():
        print(k, v["source"], [x["name"] for x in v["vectors"]])


if __name__ == "__main__":
    main()
