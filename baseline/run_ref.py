"""Times the reference's own CUDA solution (its stock ``run()``, unmodified) on one GPU with the
seeded inputs of ``fused_moe_b200.synth`` and prints one JSON object.  Single GPU only.

    python baseline/run_ref.py [--cases 1,16,64,1024,4096,16384,zipf2048] [--iters 10]

Needs ``baseline/_ref/`` (see ``baseline/build_ref.py``): the reference's torch extension and its
host module.  The extension is loaded from the build folder and handed to the host module through
its ``_ext`` global, which its loader honours (solution/python/kernel.py:27-29 of the reference),
so nothing is JIT-compiled here.  Per case: 3 warm-up calls, then ``iters`` calls timed one by one
with CUDA events, the L2 flushed by a 256 MB write before each; the median is reported.  Calls of
4096 tokens and more take the reference's lossy MxF8 sub-path by default; its exact block-scale
path (its own ``USE_MXF8=0`` switch) is timed as well.  Outputs are compared with this library's
at the contest harness's band only (|d| <= 1 + 0.3 |ref|): the reference rounds the routing logits
to bf16 and, on the MxF8 path, re-rounds the weights.
"""
from __future__ import annotations

import argparse
import glob
import importlib.util
import json
import os
import statistics
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF = os.path.join(HERE, "_ref")
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def load_reference():
    import torch  # noqa: F401  (the extension links against libtorch)
    so = sorted(glob.glob(os.path.join(REF, "build", "moe_gemm_v6_multifile*.so")))
    host = os.path.join(REF, "kernel.py")
    if not so or not os.path.isfile(host):
        return None, "baseline/_ref is not built (python baseline/build_ref.py)"
    spec = importlib.util.spec_from_file_location("moe_gemm_v6_multifile", so[0])
    ext = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ext)
    spec = importlib.util.spec_from_file_location("reference_kernel", host)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod._ext = ext
    return mod, None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--cases", default="1,16,64,1024,4096,16384,zipf2048")
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    import torch
    from fused_moe_b200 import kernel, synth
    mod, why = load_reference()
    if mod is None:
        print(json.dumps({"unavailable": why}))
        return 0
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    w = synth.make_weights(32, 0, 0, device=dev, fast_device_rng=True)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    token_seed = {1: 2, 4: 1}
    rows = []
    for case in args.cases.split(","):
        zipf = case.startswith("zipf")
        T = int(case[4:]) if zipf else int(case)
        lg, hq, hsc = (t.to(dev) for t in synth.make_tokens(T, 0, token_seed.get(T, 0)))
        bias = synth.make_bias(0, zipf=zipf).to(dev)
        ours = kernel.custom_kernel(lg, bias, hq, hsc, *w, 0, 2.5).clone()
        variants = [("stock", None)] + ([("exact_block_scale", "0")] if T >= 4096 else [])
        row = {"T": T, "zipf": zipf}
        for name, mxf8 in variants:
            if mxf8 is None:
                os.environ.pop("USE_MXF8", None)
            else:
                os.environ["USE_MXF8"] = mxf8
            try:
                for _ in range(3):
                    out = mod.run(lg, bias, hq, hsc, *w, 0, 2.5)
                torch.cuda.synchronize()
                ts = []
                for _ in range(args.iters):
                    flush.zero_()
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    out = mod.run(lg, bias, hq, hsc, *w, 0, 2.5)
                    b.record()
                    torch.cuda.synchronize()
                    ts.append(a.elapsed_time(b))
                row[name] = {"us": statistics.median(ts) * 1000.0,
                             "contest_band_vs_this_library": synth.contest_match(out, ours),
                             "parity_band_vs_this_library": synth.check_close(out, ours)[0]}
            except Exception as exc:   # the reference raises RuntimeError on unsupported shapes / CUDA errors
                row[name] = {"error": f"{type(exc).__name__}: {str(exc)[:200]}"}
                break
        os.environ.pop("USE_MXF8", None)
        rows.append(row)
    print(json.dumps({"what": "reference CUDA solution, stock run(), 32-expert slice, L2 flushed, median of "
                              f"{args.iters}", "rows": rows}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
