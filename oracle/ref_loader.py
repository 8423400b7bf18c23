"""Loads the reference's own torch check function for pinning the oracle.  TEST INFRASTRUCTURE ONLY.

``_reference_impl`` lives in experiments/fast_bench/correctness_bench.py:27-113 of the
reference project.  That file imports a cloud SDK at module level, so the function's
syntax tree is extracted and compiled on its own; nothing is copied into this repository.
The reference checkout is only present on the build machine: ``available()`` says whether
it can be found, and callers (the golden-vector generator, optional cross-checks) skip
when it cannot.
"""
from __future__ import annotations

import ast
import os

# FUSED_MOE_REFERENCE, or a checkout named "reference" beside this repository
_REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE_ROOT = os.environ.get("FUSED_MOE_REFERENCE", os.path.join(os.path.dirname(_REPO), "reference"))
_REL = "experiments/fast_bench/correctness_bench.py"


def available() -> bool:
    return os.path.isfile(os.path.join(REFERENCE_ROOT, _REL))


def load_reference_impl():
    path = os.path.join(REFERENCE_ROOT, _REL)
    with open(path) as fh:
        tree = ast.parse(fh.read())
    fn = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "_reference_impl"]
    if not fn:
        raise RuntimeError(f"_reference_impl not found in {path}")
    ns: dict = {}
    exec(compile(ast.Module(body=fn, type_ignores=[]), path, "exec"), ns)
    return ns["_reference_impl"]
