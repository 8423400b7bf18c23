"""The allocation-free routing entry point against the ordinary one, through the C ABI.

b200moe_route_static exists for hosts that may not allocate device memory inside the call
(plugin enqueue hooks, frozen-budget serving loops).  It must give exactly what b200moe_route
gives, on two calls in a row (the second call finds the previous call's histogram in the
shared scratch array and has to clear it), and must refuse batches beyond its fixed capacity.
This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from fused_moe_b200 import _capi, kernel, synth
from oracle import moe_oracle as O


def _route_static(lib, logits, bias, T, off, e_local, stream=0):
    dev = logits.device
    ids = torch.full((max(T, 1), 8), -7, dtype=torch.int32, device=dev)
    w = torch.full((max(T, 1), 8), -7.0, dtype=torch.float32, device=dev)
    counts = torch.full((e_local,), -7, dtype=torch.int32, device=dev)
    rc = lib.b200moe_route_static(logits.data_ptr(), _capi.F32, bias.data_ptr(), _capi.BF16, T, 2.5, off, e_local,
                                  ids.data_ptr(), w.data_ptr(), counts.data_ptr(), stream)
    return rc, ids[:T], w[:T], counts


@pytest.mark.gpu
def test_route_static_matches_route_on_two_calls_in_a_row():
    lib = _capi.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    bias = synth.make_bias(0).to(dev)
    # two different batches back to back: the second must not see the first one's histogram
    for T, seed, off, e_local in ((1000, 3, 32, 64), (333, 4, 0, 256)):
        logits = synth.make_tokens(T, 0, seed, hidden=128)[0].to(dev)
        rc, ids, w, counts = _route_static(lib, logits, bias, T, off, e_local)
        assert rc == 0, lib.b200moe_route_static_error()
        ref_ids, ref_w = kernel.route(logits, bias, 2.5, off, e_local, 256, 128)     # the existing entry point
        torch.cuda.synchronize()
        assert torch.equal(ids, ref_ids), "expert ids differ from b200moe_route"
        # same kernel, same inputs: the tests' tolerance for routing weights is 1e-6 relative
        np.testing.assert_allclose(w.cpu().numpy(), ref_w.cpu().numpy(), rtol=1e-6, atol=0)
        want = O.local_counts(ref_ids.cpu().numpy(), off, e_local)
        assert np.array_equal(counts.cpu().numpy(), want), "per-expert counts"


@pytest.mark.gpu
def test_route_static_rejects_oversized_batches_and_bad_arguments():
    lib = _capi.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cap = lib.b200moe_route_static_max_tokens()
    assert cap == 65536
    dummy = torch.zeros(64, dtype=torch.int32, device=dev)
    p = dummy.data_ptr()
    rc = lib.b200moe_route_static(p, _capi.F32, p, _capi.BF16, cap + 1, 2.5, 0, 32, p, p, p, 0)
    assert rc == -2
    assert b"at most 65536 tokens" in lib.b200moe_route_static_error()
    assert lib.b200moe_route_static(p, _capi.F32, p, _capi.BF16, 8, 2.5, 240, 32, p, p, p, 0) == -1
    assert lib.b200moe_route_static(p, _capi.F32, p, _capi.BF16, 8, 2.5, 0, 32, p, p, None, 0) == -1
    # an empty batch is fine and reports zero counts
    counts = torch.full((32,), 5, dtype=torch.int32, device=dev)
    assert lib.b200moe_route_static(None, _capi.F32, None, _capi.BF16, 0, 2.5, 0, 32, None, None,
                                    counts.data_ptr(), 0) == 0
    torch.cuda.synchronize()
    assert int(counts.abs().sum()) == 0
