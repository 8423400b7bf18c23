"""The C-ABI library without a GPU: it loads, exports what the header declares, and its
argument checks (which run before any CUDA call) behave as documented."""
import ctypes as C
import os
import re

import pytest
import torch

from conftest import ROOT
from fused_moe_b200 import _capi, kernel


def header_functions():
    text = open(os.path.join(ROOT, "include", "b200moe.h")).read()
    return re.findall(r"B200MOE_API\s+[\w\s\*]+?\b(b200moe_\w+)\s*\(", text)


def test_library_loads_and_exports_every_declared_symbol():
    lib = _capi.lib()
    names = header_functions()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/b200moe.h but not exported"
    assert set(names) == set(_capi.SIGNATURES), "ctypes signatures and header disagree"
    assert lib.b200moe_version() == 1
    assert lib.b200moe_status_string(0) == b"ok"
    assert b"timed out" in lib.b200moe_status_string(-5)


def test_header_cites_reference_or_says_no_counterpart():
    text = open(os.path.join(ROOT, "include", "b200moe.h")).read()
    blocks = re.split(r"\n\n", text)
    for n in header_functions():
        blk = [b for b in blocks if re.search(r"\b" + n + r"\s*\(", b)]
        assert blk, n
    assert "kernel.py:575-648" in text


def test_workspace_layout_is_aligned_ordered_and_grows_with_T():
    prev = 0
    for T in (0, 1, 8, 64, 257, 4096, 16384):
        L = _capi.workspace_layout(T, 32, 7168, 2048)
        offs = [getattr(L, f) for f, _ in _capi.WsLayout._fields_[1:21]]
        assert all(o % 256 == 0 for o in offs)
        assert offs == sorted(offs) and len(set(offs)) == len(offs)
        assert L.m_cap % 128 == 0 and L.m_cap >= min(8, 32) * T + 128
        assert L.max_tiles * 128 == L.m_cap
        assert L.n_chunks == max(1, -(-T // L.chunk_tokens))
        assert L.total_bytes >= prev
        prev = L.total_bytes
    # the 256-expert layer on one GPU at 4096 tokens fits comfortably in HBM
    assert _capi.workspace_layout(4096, 256, 7168, 2048).total_bytes < 4 * 2 ** 30


@pytest.mark.parametrize("T,e,h,i,code", [
    (-1, 32, 7168, 2048, -1), (8, 0, 7168, 2048, -1), (8, 257, 7168, 2048, -2),
    (8, 32, 7000, 2048, -2), (8, 32, 7168, 2000, -2), (8, 32, 128, 2048, -2),
])
def test_layout_rejects_bad_shapes(T, e, h, i, code):
    assert _capi.lib().b200moe_workspace_layout(T, e, h, i, None) == code


def test_entry_points_reject_bad_arguments_before_touching_cuda():
    lib = _capi.lib()
    L = _capi.workspace_layout(8, 32, 256, 128)
    buf = C.create_string_buffer(int(L.total_bytes) + 512)
    base = (C.addressof(buf) + 255) // 256 * 256
    one = C.create_string_buffer(64)
    p = C.addressof(one)
    # null pointers
    assert lib.b200moe_route(None, 0, p, 1, 8, 2.5, 0, 32, 256, 128, p, p, base, L.total_bytes, None) == -1
    # bad dtype tag
    assert lib.b200moe_route(p, 7, p, 1, 8, 2.5, 0, 32, 256, 128, p, p, base, L.total_bytes, None) == -1
    # expert slice outside the 256 experts
    assert lib.b200moe_route(p, 0, p, 1, 8, 2.5, 250, 32, 256, 128, p, p, base, L.total_bytes, None) == -1
    # workspace too small / misaligned
    assert lib.b200moe_route(p, 0, p, 1, 8, 2.5, 0, 32, 256, 128, p, p, base, 1024, None) == -3
    assert lib.b200moe_route(p, 0, p, 1, 8, 2.5, 0, 32, 256, 128, p, p, base + 8, L.total_bytes, None) == -6
    # ids stride shorter than a row
    assert lib.b200moe_count(p, 4, 8, 0, 32, 256, 128, base, L.total_bytes, None) == -1
    # EP world sizes
    assert lib.b200moe_ep_pack(p, p, p, 512, p, 1, 1, 8, 512, 3, p, p, p, None) == -2
    assert lib.b200moe_ep_pack(p, p, p, 512, p, 1, 1, 8, 256, 2, p, p, p, None) == -2
    assert lib.b200moe_ep_combine(p, p, p, 8, 512, 5, p, None) == -2
    # the peer-memory step: world size, row pitch and null buffers are checked before any CUDA call
    bases = (C.c_void_p * 2)(p, p)
    args = (bases, p, 2, 64, 7168 + 224 + 64, p, p, p, p, 32, 0, 7168, 2048, base, L.total_bytes, p, 7168, None)
    assert lib.b200moe_ep_local_experts(*args[:2], 3, *args[3:]) == -2
    assert lib.b200moe_ep_local_experts(*args[:4], 7168 + 224 + 60, *args[5:]) == -6
    assert lib.b200moe_ep_local_experts(None, *args[1:]) == -1


def test_launch_counts_per_call():
    """Kernels per layer call with the default switches: seven; calls of at most 32 tokens fuse routing, scan and
    placement; the decode GEMM1 (at most 16 tokens) also requantises; at most 8 tokens need no gather pass."""
    lib = _capi.lib()
    assert [lib.b200moe_launches_per_run(T, 32) for T in (0, 1, 8, 9, 16, 17, 32, 33, 4096)] == [0, 3, 3, 4, 4, 5, 5, 7, 7]


def test_host_entry_point_refuses_cpu_tensors_and_bad_shapes():
    from fused_moe_b200 import synth
    inp = synth.make_inputs(T=4, e_local=2, hidden=256, inter=128)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        kernel.run(*inp.args())


def test_scale_stride_resolution():
    kb, T = 4, 3
    a = torch.zeros(kb, T)
    assert kernel._scale_strides(a, T, kb) == (1, T)
    assert kernel._scale_strides(a.t(), T, kb) == (1, T)           # [T,kb] view of the same memory
    assert kernel._scale_strides(torch.zeros(T, kb), T, kb) == (kb, 1)
    sq = torch.zeros(4, 4)
    assert kernel._scale_strides(sq, 4, 4) == (1, 4)               # square: [K/128, T]
    with pytest.raises(ValueError):
        kernel._scale_strides(torch.zeros(5, 5), T, kb)
