"""Contest packaging: the solution document mirrors the reference packer's, and the TVM-FFI global
function runs the layer on DLPack tensors in destination-passing style."""
import json
import os

import numpy as np
import pytest
import torch

from conftest import golden_inputs


def test_solution_document_has_the_harness_fields(tmp_path):
    from fused_moe_b200.packaging import pack_solution
    out = tmp_path / "solution.json"
    assert pack_solution.main(["-o", str(out)]) == 0
    doc = json.loads(out.read_text())
    assert doc["definition"] == "moe_fp8_block_scale_ds_routing_topk8_ng8_kg4_e32_h7168_i2048"
    spec = doc["spec"]
    assert spec["language"] == "cuda" and spec["binding"] == "tvm-ffi" and spec["destination_passing_style"] is True
    assert spec["target_hardware"] == ["cuda"] and spec["entry_point"] == "binding.py::kernel"
    paths = {s["path"] for s in doc["sources"]}
    for need in ("binding.py", "include/b200moe.h", "fused_moe_b200/csrc/gemm.cu", "fused_moe_b200/csrc/capi.cu",
                 "fused_moe_b200/kernel.py", "fused_moe_b200/_capi.py", "fused_moe_b200/build.py"):
        assert need in paths, need
    assert all(s["content"] for s in doc["sources"])
    assert not any(p.endswith((".so", ".o")) for p in paths)


def test_binding_registers_the_global_function():
    import tvm_ffi
    from fused_moe_b200.packaging import binding
    fn = tvm_ffi.get_global_func(binding.GLOBAL_NAME)
    assert fn is not None
    # wrong arity is refused by the Python callee, as the harness would see it
    with pytest.raises(Exception):
        fn(torch.zeros(1))


@pytest.mark.gpu
def test_tvm_ffi_call_with_dlpack_tensors_matches_the_oracle():
    import tvm_ffi
    from fused_moe_b200 import synth
    from fused_moe_b200.packaging import binding
    from oracle import moe_oracle as O
    g, inp = golden_inputs("layer_small_T200_off64")
    dev = torch.device("cuda", 0)
    gi = inp.to(dev)
    out = torch.full((200, inp.hidden_states.shape[1]), float("nan"), dtype=torch.bfloat16, device=dev)
    fn = tvm_ffi.get_global_func(binding.GLOBAL_NAME)
    fn(*gi.args(), out)                      # torch tensors cross as DLPack tensors, scalars as scalars
    torch.cuda.synchronize()
    ora = O.moe_layer_torch(*inp.args())
    frac_all, frac_nz, max_abs = synth.check_close(out, ora["out"])
    assert frac_all >= 0.999 and frac_nz >= 0.999, (frac_all, frac_nz, max_abs)
    assert synth.contest_match(out, ora["out"]) >= 0.999
