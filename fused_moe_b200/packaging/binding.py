"""TVM-FFI binding of the layer for the FlashInfer-Bench harness (CUDA-language solutions).

Takes the place of the reference's binding template (solution/cuda/binding.py:13-25): the global
function ``flashinfer.kernel`` receives the ten inputs of the definition
``moe_fp8_block_scale_ds_routing_topk8_ng8_kg4_e32_h7168_i2048`` followed by the output tensor
(destination-passing style, as README.md:227-257 of the reference describes) as DLPack tensors and
plain scalars, and runs the C-ABI library on the caller's current CUDA stream.  Nothing is copied:
the tensors are re-wrapped through DLPack and the result is written into the caller's ``output``.
"""
from __future__ import annotations

import os
import sys

import torch
import tvm_ffi

_HERE = os.path.dirname(os.path.abspath(__file__))
for _cand in (os.path.dirname(os.path.dirname(_HERE)), _HERE):      # in-tree, or an unpacked solution
    if os.path.isdir(os.path.join(_cand, "fused_moe_b200")) and _cand not in sys.path:
        sys.path.insert(0, _cand)

GLOBAL_NAME = "flashinfer.kernel"


def _as_torch(x):
    """DLPack tensor -> torch view of the same memory; scalars (and 0-d tensors) pass through."""
    if isinstance(x, torch.Tensor):
        return x
    if hasattr(x, "__dlpack__"):
        return torch.from_dlpack(x)
    return x


def kernel(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
           gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset,
           routed_scaling_factor, output):
    from fused_moe_b200 import kernel as host
    args = [_as_torch(a) for a in (routing_logits, routing_bias, hidden_states, hidden_states_scale,
                                   gemm1_weights, gemm1_weights_scale, gemm2_weights, gemm2_weights_scale)]
    out = _as_torch(output)
    off = _as_torch(local_expert_offset)
    rsf = _as_torch(routed_scaling_factor)
    host.custom_kernel(*args, off, rsf, out=out)


def register(override: bool = True):
    """Registers ``kernel`` as the TVM-FFI global function the harness looks up; returns that function."""
    tvm_ffi.register_global_func(GLOBAL_NAME, kernel, override=override)
    return tvm_ffi.get_global_func(GLOBAL_NAME)


register()
