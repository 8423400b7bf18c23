"""Generates the golden vectors in this folder from the reference's own torch function.

Run on a machine that has the reference checkout (``oracle/ref_loader.py`` finds it):

    python tests/golden/make_golden.py

The reference has no stored test vectors of its own, so its check function
``_reference_impl`` (experiments/fast_bench/correctness_bench.py:27-113) is executed on
the seeded synthetic inputs of ``fused_moe_b200.synth`` and the results are stored:

* ``layer_small_*.npz``  whole-layer outputs (bf16 bits), expert ids and weights at
  reduced hidden/intermediate sizes (the function takes every extent but the routing
  constants from its arguments), for several offsets and token counts;
* ``layer_full_T<T>_ts<seed>.npz``  the full DeepSeek-V3 shape, 32 local experts;
* ``routing_ids.npz``  expert ids (uint8) of the reference's routing lines 47-61 for every
  token count of the benchmark configurations, the Zipf stress bias and the 8 EP ranks.

Inputs are not stored: they are regenerated from the seeds, and a checksum of every
input tensor is stored beside the outputs so that a generator drift is detected.
"""
from __future__ import annotations

import os
import sys
import zlib

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from fused_moe_b200 import synth  # noqa: E402
from oracle import ref_loader  # noqa: E402


def checksum(inp: synth.MoEInputs) -> np.ndarray:
    out = []
    for t in inp.args()[:8]:
        raw = t.contiguous().reshape(-1).view(torch.uint8).numpy().tobytes()
        out.append(zlib.crc32(raw))
    return np.asarray(out, dtype=np.uint64)


def reference_routing(logits: torch.Tensor, bias: torch.Tensor, rsf: float):
    """The reference function returns only the layer output, so its routing is pinned by
    issuing the same torch calls it makes (correctness_bench.py:47-61: sigmoid, topk over
    groups, topk over experts) on the same inputs; this is the reference's arithmetic in
    the reference's library, not this repository's restatement of it."""
    T = logits.shape[0]
    s = torch.sigmoid(logits.float())
    s_wb = s + bias.float()
    top2 = torch.topk(s_wb.view(T, 8, 32), k=2, dim=2).values
    scores = top2.sum(dim=2)
    groups = torch.topk(scores, k=4, dim=1).indices
    gmask = torch.zeros((T, 8), dtype=torch.bool)
    gmask.scatter_(1, groups, True)
    emask = gmask.unsqueeze(-1).expand(-1, -1, 32).reshape(T, 256)
    filtered = s_wb.masked_fill(~emask, float("-inf"))
    _, idx = torch.topk(filtered, k=8, dim=1)
    ts = s.gather(1, idx.long())
    w = ts * (rsf / (ts.sum(dim=1, keepdim=True) + 1e-20))
    return idx.to(torch.int32).numpy(), w.numpy()


def layer_case(ref_impl, name, **kw):
    inp = synth.make_inputs(**kw)
    out = ref_impl(*inp.args())
    ids, w = reference_routing(inp.routing_logits, inp.routing_bias, inp.routed_scaling_factor)
    np.savez_compressed(
        os.path.join(HERE, name),
        out_bits=out.view(torch.int16).numpy().view(np.uint16),
        ids=ids.astype(np.uint8), weights=w.astype(np.float32),
        input_crc=checksum(inp),
        params=np.asarray([kw.get("T"), kw.get("e_local", 32), kw.get("local_expert_offset", 0),
                           kw.get("seed", 0), kw.get("hidden", synth.HIDDEN),
                           kw.get("inter", synth.INTER), int(kw.get("zipf", False)),
                           kw.get("seed", 0) if kw.get("token_seed") is None else kw["token_seed"]],
                          dtype=np.int64))
    nz = int((out != 0).any(dim=1).sum())
    print(f"{name}: T={kw.get('T')} rows with local work {nz}, |out| max {out.float().abs().max():.4f}")


SMALL_CASES = {
    # name: kwargs of synth.make_inputs
    "layer_small_T64_off0": dict(T=64, e_local=32, local_expert_offset=0, seed=3, hidden=512, inter=256),
    "layer_small_T200_off64": dict(T=200, e_local=32, local_expert_offset=64, seed=3, hidden=512, inter=256),
    "layer_small_T57_off240_e16": dict(T=57, e_local=16, local_expert_offset=240, seed=5, hidden=512, inter=256),
    "layer_small_T300_e256": dict(T=300, e_local=256, local_expert_offset=0, seed=7, hidden=256, inter=128),
    "layer_small_T1_off0": dict(T=1, e_local=32, local_expert_offset=0, seed=1, hidden=512, inter=256),
    "layer_small_T513_zipf": dict(T=513, e_local=32, local_expert_offset=0, seed=2, hidden=512, inter=256, zipf=True),
}

# full DeepSeek-V3 shape, 32 local experts, weights of seed 0: (T, token seed).  Token seed 0 at
# T=8 happens to route no token to experts 0..31 (an all-zero output, kept as the empty case).
FULL_CASES = [(8, 0), (8, 1), (8, 2), (1, 1), (64, 0)]

ROUTING_CASES = [
    # (key, T, seed, rank, zipf)
    *[(f"T{T}_s0", T, 0, 0, False) for T in (1, 4, 8, 16, 64, 1024, 2048, 4096, 16384)],
    ("T1_s1", 1, 1, 0, False), ("T4_s1", 4, 1, 0, False),
    ("T2048_zipf", 2048, 0, 0, True),
    *[(f"T4096_rank{r}", 4096, 0, r, False) for r in range(1, 8)],
]


def main():
    if not ref_loader.available():
        raise SystemExit("reference checkout not found; golden vectors cannot be regenerated here")
    torch.set_num_threads(os.cpu_count() or 1)
    ref_impl = ref_loader.load_reference_impl()

    for name, kw in SMALL_CASES.items():
        layer_case(ref_impl, name, **kw)

    weights = synth.make_weights(32, 0, 0)
    for T, ts in FULL_CASES:
        layer_case(ref_impl, f"layer_full_T{T}_ts{ts}", T=T, e_local=32, local_expert_offset=0, seed=0,
                   weights=weights, token_seed=ts)

    rout = {}
    for key, T, seed, rank, zipf in ROUTING_CASES:
        logits, _, _ = synth.make_tokens(T, rank, seed, hidden=128)
        bias = synth.make_bias(seed, zipf)
        ids, w = reference_routing(logits, bias, 2.5)
        rout[key + "_ids"] = ids.astype(np.uint8)
        rout[key + "_wsum"] = np.asarray([w.astype(np.float64).sum()])
        if T <= 1024:
            rout[key + "_w"] = w.astype(np.float32)
        rout[key + "_crc"] = np.asarray([zlib.crc32(logits.numpy().tobytes()),
                                         zlib.crc32(bias.view(torch.int16).numpy().tobytes())],
                                        dtype=np.uint64)
    np.savez_compressed(os.path.join(HERE, "routing_ids.npz"), **rout)
    print("routing_ids.npz:", len(ROUTING_CASES), "cases")


if __name__ == "__main__":
    main()
