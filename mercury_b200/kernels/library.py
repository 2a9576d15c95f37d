"""The compiled kernels as a ctypes library, loaded once per process.

There is no fallback: if the library cannot be built or loaded, or no CUDA device is
present, `load()` raises and nothing of the engine runs.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

from .build import BuildError, bounds_check_wanted, build

_LIB = None

ERRORS = {
    1: "a size is outside what the kernel supports",
    2: "unknown dtype flag",
    3: "the CUDA launch failed",
    4: "a pointer or stride is misaligned",
    5: "the scratch buffer is too small",
}


class KernelError(RuntimeError):
    pass


_SIGNATURES = {
    "mb_embed": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p],
    "mb_add_rmsnorm": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                       c_float, c_int, c_void_p],
    "mb_swiglu": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "mb_rope_store": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                      c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                      c_void_p],
    "mb_gemm_simt": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int,
                     c_int, c_int, c_void_p],
    "mb_paged_attention_simt": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int,
                                c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int,
                                c_void_p],
    "mb_paged_attention_mma": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                               c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int,
                               c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p,
                               c_void_p],
    "mb_gemm_skinny": [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_float,
                       c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                       c_void_p, c_void_p, c_int, c_void_p, c_void_p],
    "mb_gemm_skinny_swiglu": [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int,
                              c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                              c_longlong, c_void_p, c_void_p],
    "mb_gemm_skinny_set_fed_min": [c_longlong],
    "mb_gemm_skinny_qkv_rope": [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_float,
                                c_int, c_void_p, c_void_p,
                                c_void_p, c_void_p, c_void_p, c_int,
                                c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "mb_gemm_tcgen05": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                        c_int, c_void_p],
    "mb_gemm_tcgen05_withheld": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                 c_longlong, c_void_p],
    "mb_gemm_tcgen05_persistent": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                   c_void_p, c_void_p],
    "mb_gemm_pair_supports": [c_int, c_int, c_int],
    "mb_gemm_pair_tiles": [c_int, c_int],
    "mb_gemm_pair": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int,
                     c_float, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "mb_paged_attention_tcgen05": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                   c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                   c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p],
    "mb_paged_attention_decode_cluster": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                          c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                          c_int, c_int, c_int, c_float, c_int, c_int, c_void_p,
                                          c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
    "mb_gemm_skinny_set_slices": [c_int, c_int],
    "mb_patch_tokens": [c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "mb_argmax": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p],
    "mb_sample": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
}


def load():
    """Build if needed, load, and declare the entry points."""
    global _LIB
    if _LIB is not None:
        return _LIB
    try:
        path = build(bounds_check=bounds_check_wanted())
    except BuildError as err:
        raise KernelError(f"the CUDA kernels could not be built: {err}") from err
    lib = ctypes.CDLL(str(path))
    for name, argtypes in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int
    lib.mb_gemm_tcgen05_supports.argtypes = [c_int, c_int, c_int]
    lib.mb_gemm_tcgen05_supports.restype = c_int
    lib.mb_check_enabled.argtypes = []
    lib.mb_check_enabled.restype = c_int
    lib.mb_check_set_limits.argtypes = [c_int, c_int, c_void_p]
    lib.mb_check_set_limits.restype = c_int
    lib.mb_check_read.argtypes = [ctypes.POINTER(c_int), c_void_p]
    lib.mb_check_read.restype = c_int
    lib.mb_set_dependent_launch.argtypes = [c_int]
    lib.mb_set_dependent_launch.restype = None
    lib.mb_gemm_skinny_supports.argtypes = [c_int, c_int, c_int]
    lib.mb_gemm_skinny_supports.restype = c_int
    lib.mb_gemm_skinny_qkv_supports.argtypes = [c_int, c_int, c_int, c_int]
    lib.mb_gemm_skinny_qkv_supports.restype = c_int
    lib.mb_attention_tcgen05_supports.argtypes = [c_int, c_int, c_int, c_int, c_int]
    lib.mb_attention_tcgen05_supports.restype = c_int
    lib.mb_attention_mma_supports.argtypes = [c_int]
    lib.mb_attention_mma_supports.restype = c_int
    lib.mb_attention_decode_raw_pays.argtypes = [c_int]
    lib.mb_attention_decode_raw_pays.restype = c_int
    lib.mb_attention_scratch_floats.argtypes = [c_int, c_int, c_int, c_int]
    lib.mb_attention_scratch_floats.restype = c_longlong
    _LIB = lib
    return lib


def check(code: int, what: str) -> None:
    if code != 0:
        raise KernelError(f"{what}: {ERRORS.get(code, f'error {code}')}")
