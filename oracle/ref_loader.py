"""Loads the reference's own torch check function for pinning the oracle.  TEST INFRASTRUCTURE ONLY.

``_reference_impl`` lives in experiments/fast_bench/correctness_bench.py:27-113 of the
reference project.  That file imports a cloud SDK at module level, so the function's
syntax tree is extracted and compiled on its own; nothing is copied into this repository.
The reference checkout is only present on the build machine; ``oracle/make_ref.py`` writes the
extracted function to the untracked ``oracle/_ref/reference_impl.py`` so that it can also be
executed elsewhere (the timed CPU arm of the benchmark).  ``available()`` says whether either
can be found, and callers (the golden-vector generator, the CPU arm, optional cross-checks)
skip when neither can.
"""
from __future__ import annotations

import ast
import os

# FUSED_MOE_REFERENCE, or a checkout named "reference" beside this repository
_REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE_ROOT = os.environ.get("FUSED_MOE_REFERENCE", os.path.join(os.path.dirname(_REPO), "reference"))
_REL = "experiments/fast_bench/correctness_bench.py"


_EXTRACTED = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "reference_impl.py")


def available() -> bool:
    return os.path.isfile(os.path.join(REFERENCE_ROOT, _REL)) or os.path.isfile(_EXTRACTED)


def source() -> str:
    """Which copy load_reference_impl() executes: "checkout", "extracted" or "none"."""
    if os.path.isfile(os.path.join(REFERENCE_ROOT, _REL)):
        return "checkout"
    return "extracted" if os.path.isfile(_EXTRACTED) else "none"


def load_reference_impl():
    path = os.path.join(REFERENCE_ROOT, _REL)
    if not os.path.isfile(path):
        path = _EXTRACTED
    with open(path) as fh:
        tree = ast.parse(fh.read())
    fn = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "_reference_impl"]
    if not fn:
        raise RuntimeError(f"_reference_impl not found in {path}")
    ns: dict = {}
    exec(compile(ast.Module(body=fn, type_ignores=[]), path, "exec"), ns)
    return ns["_reference_impl"]
