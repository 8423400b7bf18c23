"""Packs the library into a FlashInfer-Bench ``solution.json``.

    python -m fused_moe_b200.packaging.pack_solution [-o solution.json]

Same document as the reference's packer writes (scripts/pack_solution.py:83-143): name, definition,
author, description, a build spec (language, target_hardware, entry_point, dependencies, binding,
destination_passing_style) and every source file as ``{"path", "content"}``.  It is plain JSON
built from ``config.toml`` beside this file; the harness's own pydantic models are not needed.
The sources are the C ABI header, the CUDA sources, the Python host and the TVM-FFI binding; the
harness side builds them with ``python -m fused_moe_b200.build`` (nvcc, sm_100a).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

try:
    import tomllib
except ModuleNotFoundError:      # Python < 3.11
    import tomli as tomllib

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
ROOT = os.path.dirname(PKG)

HOST_FILES = ("__init__.py", "_capi.py", "build.py", "kernel.py")


def collect_sources():
    files = [os.path.join(ROOT, "include", "b200moe.h")]
    csrc = os.path.join(PKG, "csrc")
    files += [os.path.join(csrc, f) for f in sorted(os.listdir(csrc)) if f.endswith((".cu", ".cuh"))]
    files += [os.path.join(PKG, f) for f in HOST_FILES]
    out = []
    for path in files:
        with open(path) as fh:
            out.append({"path": os.path.relpath(path, ROOT).replace(os.sep, "/"), "content": fh.read()})
    with open(os.path.join(HERE, "binding.py")) as fh:
        out.append({"path": "binding.py", "content": fh.read()})
    return out


def build_solution() -> dict:
    with open(os.path.join(HERE, "config.toml"), "rb") as fh:
        cfg = tomllib.load(fh)
    sol, build = cfg["solution"], cfg["build"]
    if build["language"] != "cuda":
        raise ValueError("this packer writes CUDA-language solutions only")
    return {
        "name": sol["name"],
        "definition": sol["definition"],
        "author": sol["author"],
        "description": sol.get("description", f"Custom kernel for {sol['definition']}"),
        "spec": {
            "language": build["language"],
            "target_hardware": ["cuda"],
            "entry_point": build["entry_point"],
            "dependencies": [],
            "destination_passing_style": bool(build.get("destination_passing_style", True)),
            "binding": build.get("binding", "tvm-ffi"),
        },
        "sources": collect_sources(),
    }


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("-o", "--output", default=os.path.join(ROOT, "solution.json"))
    args = ap.parse_args(argv)
    doc = build_solution()
    with open(args.output, "w") as fh:
        json.dump(doc, fh, indent=2)
    print(f"Solution packed: {args.output} ({len(doc['sources'])} files, entry point {doc['spec']['entry_point']})")
    return 0


if __name__ == "__main__":
    sys.exit(main())
