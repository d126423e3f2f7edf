"""ctypes binding of libbwmoe.so (the C ABI declared in include/bwmoe.h)."""

from __future__ import annotations

import ctypes as C
import threading
from pathlib import Path

import os

_HERE = Path(__file__).resolve().parent
# BWMOE_LIBRARY selects another build of the same library (A/B timing of kernel variants)
_LIB_PATH = Path(os.environ["BWMOE_LIBRARY"]) if os.environ.get("BWMOE_LIBRARY") else _HERE / "libbwmoe.so"
_lock = threading.Lock()
_lib = None


class BwmoeError(RuntimeError):
    """A libbwmoe call failed; ``code`` is the negative BWMOE_ERR_* value."""

    def __init__(self, code: int, message: str):
        super().__init__(f"libbwmoe error {code}: {message}")
        self.code = code


def library_path() -> Path:
    return _LIB_PATH


_vp, _i, _sz, _fp, _ip = C.c_void_p, C.c_int, C.c_size_t, C.c_void_p, C.c_void_p

# name -> (restype, argtypes); every symbol the header declares
SIGNATURES = {
    "bwmoe_version": (_i, []),
    "bwmoe_set_sm_reserve": (_i, [_i]),
    "bwmoe_invalidate": (_i, []),
    "bwmoe_launch_count": (C.c_longlong, []),
    "bwmoe_last_error": (_i, [C.c_char_p, _sz]),
    "bwmoe_workspace_bytes": (_sz, [_i] * 5),
    "bwmoe_workspace_bytes_host": (_sz, [_i] * 5),
    "bwmoe_workspace_view": (_i, [_vp, _i, _i, _i, _i, _i, _i, C.POINTER(_vp), C.POINTER(_sz)]),
    "bwmoe_read_status": (_i, [_vp, _vp, C.POINTER(C.c_int32)]),
    "bwmoe_router_scratch_bytes": (_sz, [_i] * 4),
    "bwmoe_router": (_i, [_vp, _vp, _i, _i, _i, _i, _fp, _ip, _fp, _vp, _sz, _vp]),
    "bwmoe_router_scratch_bytes_as": (_sz, [_i] * 5),
    "bwmoe_router_as": (_i, [_vp, _vp, _i, _i, _i, _i, _i, _fp, _ip, _fp, _vp, _sz, _vp]),
    "bwmoe_moe_forward": (_i, [_vp] * 5 + [_fp] * 3 + [_i] * 5 + [_vp, _vp, _sz, _vp]),
    "bwmoe_moe_forward_flags": (_i, [_vp] * 5 + [_fp] * 3 + [_i] * 5 + [_vp, _vp, _sz, _vp, C.c_uint]),
    "bwmoe_moe_forward_ex": (_i, [_vp] * 5 + [_fp] * 3 + [_i] * 5 + [C.c_float, _vp, _vp, _vp, _sz, _vp]),
    "bwmoe_workspace_bytes_shared": (_sz, [_i] * 6),
    "bwmoe_moe_forward_shared": (_i, [_vp] * 5 + [_fp] * 3 + [_i] * 6 + [C.c_float, _vp, _vp, _sz, _vp]),
    "bwmoe_dense_mlp": (_i, [_vp] * 4 + [_fp] * 3 + [_i] * 3 + [_vp, _vp, _sz, _vp]),
    "bwmoe_moe_forward_routed": (_i, [_vp, _fp, _ip] + [_vp] * 3 + [_fp] * 3 + [_i] * 5 + [_vp, _vp, _sz, _vp]),
    "bwmoe_moe_forward_routed_remap": (_i, [_vp, _fp, _ip, _ip, _i] + [_vp] * 3 + [_fp] * 3 + [_i] * 5
                                       + [_vp, _vp, _sz, _vp]),
    "bwmoe_moe_forward_block_routed": (_i, [_vp, _fp, _ip, _ip, _i] + [_vp] * 3 + [_fp] * 3 + [_i] * 5
                                       + [_vp, _vp, _sz, _vp]),
    "bwmoe_moe_forward_host": (_i, [_vp] * 5 + [_fp] * 3 + [_i] * 5 + [_vp, _vp, _sz, _vp]),
    "bwmoe_workspace_bytes_block": (_sz, [_i] * 5),
    "bwmoe_workspace_view_block": (_i, [_vp, _i, _i, _i, _i, _i, _i, C.POINTER(_vp), C.POINTER(_sz)]),
    "bwmoe_moe_forward_block": (_i, [_vp] * 5 + [_fp] * 3 + [_i] * 5 + [_vp, _vp, _sz, _vp]),
    "bwmoe_gather_quant_group": (_i, [_vp, _ip, _i, _i, _i, _vp, _fp, _vp]),
    "bwmoe_gateup_swiglu_block": (_i, [_vp, _fp, _ip, _vp, _vp, _fp, _fp, _i, _i, _i, _i, _vp, _fp, _ip, _vp]),
    "bwmoe_down_block": (_i, [_vp, _fp, _ip, _vp, _fp, _i, _i, _i, _i, _vp, _ip, _vp]),
    "bwmoe_plan_scratch_bytes": (_sz, [_i] * 3),
    "bwmoe_permute_plan": (_i, [_ip, _fp, _i, _i, _i, _ip, _ip, _ip, _ip, _fp, _ip, _vp, _vp]),
    "bwmoe_permute_plan_static": (_i, [_ip, _fp, _i, _i, _i, _ip, _ip, _ip, _ip, _fp, _ip, _vp]),
    "bwmoe_segment_scales": (_i, [_fp, _ip, _i, _fp, _vp]),
    "bwmoe_gather_quant": (_i, [_vp, _ip, _ip, _fp, _i, _i, _i, _vp, _vp]),
    "bwmoe_gemm_scratch_bytes": (_sz, [_i] * 4),
    "bwmoe_gateup_swiglu": (_i, [_vp, _ip, _fp, _vp, _vp, _fp, _fp, _i, _i, _i, _i, _vp, _fp, _ip, _vp, _vp]),
    "bwmoe_requant": (_i, [_vp, _ip, _fp, _i, _i, _vp, _vp]),
    "bwmoe_requant_segments": (_i, [_vp, _ip, _fp, _i, _i, _vp, _vp]),
    "bwmoe_down": (_i, [_vp, _ip, _fp, _vp, _fp, _i, _i, _i, _i, _vp, _ip, _vp, _vp]),
    "bwmoe_combine": (_i, [_vp, _ip, _fp, _i, _i, _i, _vp, _vp]),
    "bwmoe_ep_maps": (_i, [_ip, _ip, _i, _i, _i, _ip, _ip, _ip, _ip, _vp]),
    "bwmoe_down_peers": (_i, [_vp, _ip, _fp, _vp, _fp, _i, _i, _i, _i, _ip, _ip, C.POINTER(C.c_void_p), _i, _ip, _vp]),
    "bwmoe_down_block_peers": (_i, [_vp, _fp, _ip, _vp, _fp, _i, _i, _i, _i, _ip, _ip, C.POINTER(C.c_void_p), _i, _ip, _vp]),
    "bwmoe_scatter_rows_group_peers": (_i, [_vp, _fp, _ip, _ip, _ip, _i, _i, _i, _i, C.POINTER(C.c_void_p),
                                           C.POINTER(C.c_void_p), _i, _i, _ip, _vp]),
    "bwmoe_scatter_quant_peers": (_i, [_vp, _ip, _ip, _fp, _ip, _i, _i, _i, _i, C.POINTER(C.c_void_p), _i, _i, _ip,
                                       _vp]),
    "bwmoe_combine_peers": (_i, [C.POINTER(C.c_void_p), _i, _ip, _ip, _fp, _ip, _i, _i, _i, _i, _vp, _vp]),
}


def lib() -> C.CDLL:
    """Load the shared library once.  Raises if it has not been built: there is
    no other implementation to fall back to."""
    global _lib
    with _lock:
        if _lib is None:
            if not _LIB_PATH.exists():
                raise BwmoeError(-5, f"{_LIB_PATH} is missing: run `python blackwell-moe_b200/build.py` "
                                     "(or __graft_entry__.build()) first")
            handle = C.CDLL(str(_LIB_PATH))
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(handle, name)      # AttributeError if the export is missing
                fn.restype, fn.argtypes = res, args
            _lib = handle
    return _lib


def last_error() -> str:
    buf = C.create_string_buffer(512)
    lib().bwmoe_last_error(buf, 512)
    return buf.value.decode(errors="replace")


def check(rc: int) -> None:
    if rc != 0:
        msg = last_error()
        if rc in (-1, -2, -3, -6):
            raise ValueError(f"libbwmoe error {rc}: {msg}")
        raise BwmoeError(rc, msg)
