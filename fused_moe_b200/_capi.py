"""ctypes binding of ``libb200moe.so`` (the C ABI declared in ``include/b200moe.h``).

There is no fallback: if the shared library has not been built, importing a symbol
raises with the build command.  Nothing here touches torch; tensors cross as raw
device pointers.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libb200moe.so")

OK = 0
F32, BF16 = 0, 1

STATUS_NAMES = {
    0: "ok", -1: "invalid argument", -2: "unsupported shape", -3: "workspace too small",
    -4: "CUDA call failed", -5: "device-side wait timed out", -6: "misaligned pointer or stride",
}


class MoEError(RuntimeError):
    def __init__(self, status: int, what: str, extra: str = ""):
        self.status = status
        msg = f"{what}: b200moe status {status} ({STATUS_NAMES.get(status, 'unknown')})"
        if extra:
            msg += f" [{extra}]"
        super().__init__(msg)


class WsLayout(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in (
        "total_bytes", "status", "meta", "splitk_count", "tile_done", "chunk_counts", "chunk_base", "expert_count",
        "expert_row0", "tile_expert", "row_token", "row_weight", "a_packed", "a_scale", "act",
        "row_amax", "act_q", "row_scale", "tok_rows", "topk_ids", "topk_w", "trace", "splitk_scratch",
        "ep_segments")] + [
        (n, C.c_int32) for n in ("m_cap", "max_tiles", "n_chunks", "chunk_tokens")]


# name -> (restype, argtypes); mirrors include/b200moe.h one to one
_P, _I, _L, _F, _Z = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t
SIGNATURES = {
    "b200moe_version": (_I, []),
    "b200moe_status_string": (C.c_char_p, [_I]),
    "b200moe_last_cuda_error": (C.c_char_p, []),
    "b200moe_workspace_layout": (_I, [_I, _I, _I, _I, C.POINTER(WsLayout)]),
    "b200moe_route": (_I, [_P, _I, _P, _I, _I, _F, _I, _I, _I, _I, _P, _P, _P, _Z, _P]),
    "b200moe_route_static": (_I, [_P, _I, _P, _I, _I, _F, _I, _I, _P, _P, _P, _P]),
    "b200moe_route_static_max_tokens": (_I, []),
    "b200moe_route_static_error": (C.c_char_p, []),
    "b200moe_count": (_I, [_P, _L, _I, _I, _I, _I, _I, _P, _Z, _P]),
    "b200moe_experts": (_I, [_P, _L, _P, _L, _P, _L, _P, _L, _L, _P, _P, _P, _P,
                             _I, _I, _I, _I, _I, _P, _Z, _P, _L, _P]),
    "b200moe_run": (_I, [_P, _I, _P, _I, _P, _L, _P, _L, _L, _P, _P, _P, _P,
                         _I, _I, _I, _F, _I, _I, _P, _Z, _P, _L, _P]),
    "b200moe_read_status": (_I, [_P, _P, C.POINTER(C.c_int32)]),
    "b200moe_set_status_mirror": (_I, [_P]),
    "b200moe_profile_next_gemm1": (_I, [_P, _P]),
    "b200moe_selftest_wait_timeout": (_I, [_P, _P]),
    "b200moe_launches_per_run": (_I, [_I, _I]),
    "b200moe_ep_pack": (_I, [_P, _P, _P, _L, _P, _L, _L, _I, _I, _I, _P, _P, _P, _P]),
    "b200moe_ep_combine": (_I, [_P, _P, _P, _I, _I, _I, _P, _P]),
    "b200moe_ep_local_experts": (_I, [_P, _P, _I, _I, _L, _P, _P, _P, _P, _I, _I, _I, _I, _P, _Z, _P, _L, _P]),
    "b200moe_ep_combine_peers": (_I, [_P, _P, _P, _I, _I, _I, _P, _P]),
}

_lib = None


def lib() -> C.CDLL:
    """The loaded library; raises if it was never built (no CPU or torch fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.isfile(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m fused_moe_b200.build` "
                "(needs nvcc; there is no fallback path)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)   # AttributeError if the header and the library diverge
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status: int, what: str) -> None:
    if status != OK:
        extra = ""
        if status == -4:
            extra = lib().b200moe_last_cuda_error().decode(errors="replace")
        raise MoEError(status, what, extra)


def workspace_layout(T: int, e_local: int, hidden: int, inter: int) -> WsLayout:
    L = WsLayout()
    check(lib().b200moe_workspace_layout(T, e_local, hidden, inter, C.byref(L)), "workspace_layout")
    return L
