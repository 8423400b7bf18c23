"""Recipe: extracts the reference's own torch check function into ``oracle/_ref/``.  TEST INFRASTRUCTURE ONLY.

    python oracle/make_ref.py [--reference /path/to/fused-moe]

``_reference_impl`` (experiments/fast_bench/correctness_bench.py:27-113 of the reference project)
is pure torch, but its file imports a cloud SDK at module level, so the function's source text is
cut out by syntax tree and written, unmodified, to ``oracle/_ref/reference_impl.py``.  That folder
is not tracked by git; it exists so that the function can be executed where the reference
checkout is absent (the timed CPU arm of ``bench.py`` on a GPU machine).  Nothing of the product
path reads it.
"""
from __future__ import annotations

import argparse
import ast
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "reference_impl.py")
REL = os.path.join("experiments", "fast_bench", "correctness_bench.py")


def find_reference(arg=None):
    for cand in (arg, os.environ.get("FUSED_MOE_REFERENCE"),
                 os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")):
        if cand and os.path.isfile(os.path.join(cand, REL)):
            return cand
    return None


def make(reference=None) -> str | None:
    ref = find_reference(reference)
    if ref is None:
        return None
    path = os.path.join(ref, REL)
    with open(path) as fh:
        text = fh.read()
    fn = [n for n in ast.parse(text).body if isinstance(n, ast.FunctionDef) and n.name == "_reference_impl"]
    if not fn:
        raise RuntimeError(f"_reference_impl not found in {path}")
    seg = ast.get_source_segment(text, fn[0])
    os.makedirs(OUT_DIR, exist_ok=True)
    with open(OUT, "w") as fh:
        fh.write("# Extracted verbatim by oracle/make_ref.py from the reference project's\n"
                 f"# {REL.replace(os.sep, '/')} (lines {fn[0].lineno}-{fn[0].end_lineno}).  Not tracked by git.\n")
        fh.write(seg + "\n")
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None)
    out = make(ap.parse_args().reference)
    print(out if out else "reference checkout not found; nothing written")
    sys.exit(0)
