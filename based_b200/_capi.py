"""ctypes binding of ``libbased_b200.so`` (declared in ``include/based_b200.h``).

The library is loaded lazily on first use.  A missing library is an error, never a reason
to fall back to another implementation.
"""
import ctypes
import os
from ctypes import c_float, c_int, c_int32, c_int64, c_void_p, POINTER, c_char_p

from .build import library_path

BASED_F32 = 0
BASED_BF16 = 1
IMPL_AUTO = 0
IMPL_SIMT = 1
IMPL_TCGEN05 = 2

_I64P = POINTER(c_int64)

# name -> (restype, argtypes); every symbol the header declares
SIGNATURES = {
    "based_b200_version": (c_int, []),
    "based_error_string": (c_char_p, [c_int]),
    "based_read_status": (c_int, [POINTER(ctypes.c_uint), c_int]),
    "based_linattn_prefill": (c_int, [c_void_p] * 6 + [c_int] * 5 + [_I64P] * 4 + [c_int, c_int, c_float, c_int, c_void_p]),
    "based_linattn_prefill_segments": (c_int, [c_int] * 3),
    "based_linattn_prefill_scratch_bytes": (ctypes.c_size_t, [c_int] * 5),
    "based_linattn_prefill_split": (c_int, [c_void_p] * 6 + [c_int] * 5 + [_I64P] * 4
                                    + [c_int, c_float, c_int, c_void_p, ctypes.c_size_t, c_void_p]),
    "based_linattn_prefill_split_static": (c_int, [c_void_p] * 6 + [c_int] * 5 + [_I64P] * 4
                                           + [c_int, c_float, c_int, c_void_p]),
    "based_linattn_decode": (c_int, [c_void_p] * 6 + [c_int] * 4 + [_I64P] * 4 + [c_int, c_int, c_float, c_void_p]),
    "based_swa_prefill": (c_int, [c_void_p] * 4 + [c_int] * 4 + [_I64P] * 4 + [c_int, c_float, c_int, c_int, c_void_p]),
    "based_rotary_apply": (c_int, [c_void_p] + [c_int] * 4 + [_I64P, c_void_p, c_void_p, c_int, POINTER(c_int32), c_int,
                                   c_int, c_void_p]),
    "based_swa_decode": (c_int, [c_void_p] * 5 + [POINTER(c_int32), c_int, c_void_p, c_void_p, c_int]
                         + [c_int] * 4 + [_I64P] * 4 + [c_int, c_float, c_int, c_void_p]),
    "based_gated_conv_prefill": (c_int, [c_void_p] * 6 + [c_int] * 4 + [_I64P] * 3 + [c_int, c_int, c_void_p]),
    "based_gated_conv_step": (c_int, [c_void_p] * 6 + [c_int] * 3 + [c_int64] * 3 + [c_int, c_int, c_void_p]),
    "based_add_rmsnorm": (c_int, [c_void_p] * 6 + [c_int64, c_int] + [c_int64] * 4 + [c_float, c_int, c_int, c_int, c_int, c_void_p]),
    "based_gated_act": (c_int, [c_void_p] * 3 + [c_int64, c_int] + [c_int64] * 3 + [c_int, c_int, c_void_p]),
    "based_decode_linear": (c_int, [c_void_p] * 4 + [c_int] * 3 + [c_int64] * 2 + [c_int, c_int]
                            + [c_void_p] * 3 + [c_int, c_int, c_void_p]),
    "based_tp_outproj_workspace_bytes": (ctypes.c_size_t, [c_int] * 3),
    "based_tp_outproj_workspace_init": (c_int, [c_void_p, ctypes.c_size_t, c_void_p]),
    "based_tp_outproj_allreduce": (c_int, [c_void_p] * 4 + [c_int] * 3 + [c_int64] * 2 + [POINTER(c_void_p), c_int, c_int,
                                                                                          c_int, c_void_p]),
    "based_tp_outproj_allreduce_emulated": (c_int, [POINTER(c_void_p), POINTER(c_void_p), c_void_p, POINTER(c_void_p)]
                                            + [c_int] * 3 + [c_int64] * 2 + [POINTER(c_void_p), c_int, c_int, c_void_p]),
    "based_rotary_qkv_cache": (c_int, [c_void_p] + [c_int] * 4 + [_I64P, c_void_p, c_void_p, c_void_p, _I64P, c_void_p]),
}

_lib = None


class BasedLibraryError(RuntimeError):
    pass


def lib():
    global _lib
    if _lib is None:
        path = library_path()
        if not os.path.exists(path):
            raise BasedLibraryError(
                f"{path} is missing: build it with `python -m based_b200.build` "
                "(the kernels have no CPU or eager fallback)")
        handle = ctypes.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def read_status(reset: bool = True) -> int:
    """The tensor-core kernels' status word (0 = no bounded wait has expired); synchronises."""
    out = ctypes.c_uint(0)
    check(lib().based_read_status(ctypes.byref(out), 1 if reset else 0), "based_read_status")
    return out.value


def pointers(vals):
    """A C array of void* from integers (device addresses)."""
    return (c_void_p * len(vals))(*[int(v) for v in vals])


def strides(*vals):
    return (c_int64 * len(vals))(*[int(v) for v in vals])


def check(code, what):
    if code != 0:
        msg = lib().based_error_string(int(code)).decode()
        raise BasedLibraryError(f"{what} failed with code {code}: {msg}")
