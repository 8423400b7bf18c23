"""Builds the reference's own CUDA solution (its two .cu files, unmodified, compiled where they
lie in the reference checkout) into the git-ignored ``baseline/_ref/`` so that its stock
``run()`` can be timed on the same GPU and the same seeded inputs as this library.

    python baseline/build_ref.py [--reference /path/to/fused-moe]

Outputs (nothing of this is tracked by git):
    baseline/_ref/build/moe_gemm_v6_multifile.so   the reference's torch extension, sm_100a
    baseline/_ref/kernel.py                        the reference's host module (solution/python/kernel.py)

The reference JIT-builds the same extension on first use (solution/python/kernel.py:27-126) but
only looks for CUTLASS under ~/.local and /opt/conda; here the CUTLASS 4.x headers come from the
flashinfer wheel.  ``baseline/run_ref.py`` pre-seeds ``kernel._ext`` with the built module, which
``_get_ext`` honours (kernel.py:27-29).  The build takes about 12 minutes on 8 cores.
"""
from __future__ import annotations

import argparse
import os
import shutil
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def find_reference(arg):
    for cand in (arg, os.environ.get("FUSED_MOE_REFERENCE"),
                 os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")):
        if cand and os.path.isfile(os.path.join(cand, "solution", "python", "kernel.py")):
            return cand
    return None


def cutlass_includes():
    import flashinfer
    root = os.path.join(os.path.dirname(flashinfer.__file__), "data", "cutlass")
    inc = [os.path.join(root, "include"), os.path.join(root, "tools", "util", "include")]
    for p in inc:
        if not os.path.isdir(p):
            raise RuntimeError(f"CUTLASS headers not found at {p}")
    return inc


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None)
    args = ap.parse_args()
    ref = find_reference(args.reference)
    if ref is None:
        print("reference checkout not found; nothing built")
        return 1
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    import torch.utils.cpp_extension as ce
    build_dir = os.path.join(OUT, "build")
    os.makedirs(build_dir, exist_ok=True)
    src = os.path.join(ref, "solution", "python")
    t0 = time.time()
    ce.load(name="moe_gemm_v6_multifile",
            sources=[os.path.join(src, "moe_gemm.cu"), os.path.join(src, "moe_fused.cu")],
            extra_include_paths=cutlass_includes(),
            extra_cuda_cflags=["-O3", "--std=c++17", "-arch=sm_100a", "--expt-relaxed-constexpr", "-DNDEBUG",
                               "--threads=4"],
            build_directory=build_dir, verbose=True, is_python_module=False)
    shutil.copyfile(os.path.join(src, "kernel.py"), os.path.join(OUT, "kernel.py"))
    print(f"built in {time.time() - t0:.0f} s -> {build_dir}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
