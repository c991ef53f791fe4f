"""ctypes bindings of the CUDA libraries, loaded (and compiled) on first use.

Every exported kernel launcher returns 0, a CUDA error code, or a negative
refusal code; ``check`` turns anything but 0 into an exception.  There is no
fallback: on a machine without the compiler or without a GPU the call fails.
"""
from __future__ import annotations

import ctypes
import threading

from .build import build_library

F32, BF16 = 0, 1

_c = ctypes
_vp, _i, _f, _ll = _c.c_void_p, _c.c_int, _c.c_float, _c.c_longlong

# library -> {function: argtypes}
_SIGNATURES = {
    "elementwise": {
        "mstar_embed_rows": [_vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _vp],
        "mstar_scale_softcap": [_vp, _ll, _f, _f, _vp],
        "mstar_add_rmsnorm": [_vp, _vp, _vp, _i, _vp, _i, _i, _i, _f, _f, _i, _vp],
        "mstar_gather_add_rows": [_vp, _vp, _i, _vp, _vp, _i, _i, _vp],
        "mstar_silu_mul": [_vp, _vp, _i, _i, _i, _vp],
        "mstar_convert": [_vp, _i, _vp, _i, _ll, _vp],
        "mstar_rope_kv_write": [_vp, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i,
                                _i, _i, _vp],
    },
    "attention_generic": {
        "mstar_paged_attention_generic": [_vp, _i, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i,
                                          _i, _i, _f, _i, _vp],
    },
    "attention_decode": {
        "mstar_make_kv_tensor_map": [_vp, _vp, _ll, _i, _i, _i],
        "mstar_paged_decode_attention_bf16_tma": [_vp, _vp, _i, _vp, _vp, _vp, _i, _vp, _vp, _i, _i,
                                                  _i, _i, _i, _f, _i, _i, _i, _vp, _vp, _vp],
        "mstar_paged_decode_attention_bf16": [_vp, _i, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i,
                                              _i, _i, _i, _f, _i, _i, _vp, _vp],
    },
    "attention_prefill": {
        "mstar_paged_prefill_attention_bf16": [_vp, _vp, _i, _vp, _vp, _vp, _i, _vp, _vp, _i, _i,
                                               _i, _i, _i, _i, _i, _i, _f, _vp, _vp],
    },
    "attention_prefill_tc": {
        "mstar_paged_prefill_attention_tc": [_vp, _vp, _i, _i, _vp, _vp, _i, _vp, _vp, _i, _i, _i,
                                             _i, _i, _i, _i, _f, _vp, _vp],
    },
    "gemm_f32": {
        "mstar_sgemm_nt": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp],
    },
    "gemm_smallm_bulk": {
        "mstar_gemm_smallm_bulk_bf16": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp],
        "mstar_qkv_rope_write_bulk_bf16": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i,
                                           _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp],
    },
    "gemm_tcgen05": {
        "mstar_gemm_tcgen05_bf16": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp],
        "mstar_gemm_tcgen05_gated_bf16": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp],
    },
    "gemm_skinny": {
        "mstar_gemm_skinny_bf16": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp],
    },
    "sampling": {
        "mstar_sample": [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
        "mstar_argmax": [_vp, _i, _i, _i, _vp, _vp, _vp, _vp],
    },
}

_libs: dict = {}
_lock = threading.Lock()


class KernelError(RuntimeError):
    pass


def register_signatures(library: str, signatures: dict) -> None:
    """Let a further library (added to ``build.LIBRARIES``) declare its functions."""
    _SIGNATURES.setdefault(library, {}).update(signatures)
    _libs.pop(library, None)


def get(library: str):
    lib = _libs.get(library)
    if lib is not None:
        return lib
    with _lock:
        lib = _libs.get(library)
        if lib is not None:
            return lib
        path = build_library(library)
        lib = ctypes.CDLL(str(path))
        for fn, argtypes in _SIGNATURES.get(library, {}).items():
            f = getattr(lib, fn)
            f.argtypes = argtypes
            f.restype = _i
        _libs[library] = lib
        return lib


def loaded_libraries() -> dict:
    return {name: lib._name for name, lib in _libs.items()}


_launches = 0


def launch_count() -> int:
    """Kernel launches of this package's own libraries since the process began."""
    return _launches


def add_launches(n: int) -> None:
    """Account for kernels launched by replaying a captured CUDA graph."""
    global _launches
    _launches += n


def check(code: int, what: str) -> None:
    global _launches
    _launches += 1
    if code == 0:
        return
    if code < 0:
        raise KernelError(f"{what}: the kernel refuses this shape (code {code})")
    raise KernelError(f"{what}: CUDA error {code}")
