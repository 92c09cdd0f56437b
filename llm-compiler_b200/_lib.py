"""ctypes binding of libb200serve.so (declared in include/b200_serve.h).

The library is the only compute path of this package: loading fails loudly when the
shared object is missing and nothing falls back to PyTorch, Triton or the CPU.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_double, c_int, c_int32, c_int64, c_void_p
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
# B200_LIBRARY_PATH: another build of the same library (for instance the -DB200_TRACE one)
LIBRARY_PATH = Path(os.environ.get("B200_LIBRARY_PATH", PACKAGE_DIR / "libb200serve.so"))

F32, BF16, F16 = 0, 1, 2
MODE_FAST, MODE_PYTORCH_COMPATIBLE = 0, 1
EPILOGUE_NONE, EPILOGUE_RESIDUAL, EPILOGUE_SWIGLU = 0, 1, 2

STATUS_KV_OVERFLOW = 1
STATUS_LENGTH_OVER_MASK = 2
STATUS_BAD_TOKEN_ID = 4
STATUS_BAD_POSITION = 8
STATUS_WAIT_TIMEOUT = 16

LAUNCH_PROGRAMMATIC = 1
LAUNCH_CONSTANT_WEIGHTS = 2
LAUNCH_STABLE_KV_PREFIX = 4
LAUNCH_LINEAR_WARP_LEVEL = 8
LAUNCH_PREFILL_WARP_LEVEL = 16

ERR_BAD_ARGUMENT, ERR_UNSUPPORTED, ERR_ALIGNMENT = -1, -2, -3
ERR_WORKSPACE, ERR_LAUNCH, ERR_TOO_LARGE = -4, -5, -6


class B200LibraryError(RuntimeError):
    """libb200serve.so is missing or does not export the declared ABI."""


_I64P = POINTER(c_int64)

# What b200_abi_version() of a matching library returns (bumped with every signature change).
ABI_VERSION = 104

# name -> (restype, argtypes); mirrors include/b200_serve.h one to one
SIGNATURES = {
    "b200_abi_version": (c_int, []),
    "b200_error_string": (c_char_p, [c_int]),
    "b200_debug_set_waits": (c_int64, [c_int64, c_int]),
    "b200_set_launch_mode": (c_int, [c_int]),
    "b200_get_launch_mode": (c_int, []),
    "b200_kv_store": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                              c_int64, c_int64, c_int64, _I64P, _I64P, c_int, c_void_p, c_void_p]),
    "b200_rope": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                          c_int64, c_int64, c_int64, c_int64, _I64P, _I64P, _I64P, _I64P, c_int,
                          c_void_p]),
    "b200_rope_kv_store": (c_int, [c_void_p] * 9 + [c_int64] * 12 + [c_int, c_void_p, c_void_p]),
    "b200_rope_table": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int,
                                c_void_p]),
    "b200_rms_norm": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_double,
                              c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "b200_decode_attention_workspace_bytes": (c_int64, [c_int64] * 6),
    "b200_decode_attention": (c_int, [c_void_p] * 6 + [c_int64] * 9 + [c_int, c_double, c_int,
                                                                       c_int, c_int64, c_int64,
                                                                       c_void_p, c_int64, c_void_p,
                                                                       c_void_p]),
    "b200_decode_attention_ordered": (c_int, [c_void_p] * 7 + [c_int64] * 9 +
                                      [c_int, c_double, c_int, c_int, c_int64, c_int64,
                                       c_void_p, c_int64, c_void_p, c_void_p]),
    "b200_decode_attention_static_scratch_bytes": (c_int64, []),
    "b200_decode_attention_static_scratch": (c_int, [c_void_p] * 6 + [c_int64] * 9 +
                                             [c_int, c_double, c_int, c_int, c_int64, c_int64,
                                              c_void_p, c_void_p]),
    "b200_paged_kv_store": (c_int, [c_void_p] * 6 + [c_int64] * 7 + [_I64P, _I64P, c_int, c_void_p,
                                                                     c_void_p]),
    "b200_paged_decode_attention": (c_int, [c_void_p] * 7 + [c_int64] * 11 +
                                    [c_int, c_double, c_int, c_int64, c_int64, c_void_p, c_int64,
                                     c_void_p, c_void_p]),
    "b200_prefill_attention_workspace_bytes": (c_int64, [c_int64, c_int64]),
    "b200_prefill_attention": (c_int, [c_void_p] * 5 + [c_int64] * 5 + [_I64P] * 4 +
                               [c_int, c_double, c_int, c_int, c_int, c_void_p, c_int64, c_void_p,
                                c_void_p]),
    "b200_classify_causal_mask": (c_int, [c_void_p, c_int64, c_int64, _I64P, c_int, c_void_p,
                                          c_void_p]),
    "b200_linear_workspace_bytes": (c_int64, [c_int64, c_int64, c_int64, c_int, c_int]),
    "b200_linear": (c_int, [c_void_p] * 5 + [c_int64] * 4 + [c_int, c_int, c_void_p, c_int64,
                                                              c_void_p, c_void_p]),
    "b200_linear_partial_splits": (c_int64, [c_int64, c_int64, c_int64]),
    "b200_linear_partial": (c_int, [c_void_p] * 4 + [c_int64] * 5 + [c_void_p, c_void_p]),
    "b200_reduce_residual_rms_norm": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_int64, c_int64, c_double, c_int, c_void_p]),
    "b200_reduce_rope_kv_store": (c_int, [c_void_p, c_int64] + [c_void_p] * 7 + [c_int64] * 5 +
                                  [c_void_p, c_void_p]),
    "b200_qkv_decode_attention": (c_int, [c_void_p, c_int64] + [c_void_p] * 7 +
                                  [c_int64] * 6 + [c_double, c_int64, c_int64, c_int64, c_void_p,
                                                   c_int64, c_double, c_void_p, c_void_p, c_int64,
                                                   c_void_p, c_void_p]),
    "b200_paged_qkv_decode_attention": (c_int, [c_void_p, c_int64] + [c_void_p] * 8 +
                                        [c_int64] * 8 + [c_double, c_int64, c_int64, c_int64,
                                                         c_void_p, c_int64, c_double, c_void_p,
                                                         c_void_p, c_int64, c_void_p, c_void_p]),
    "b200_scale_columns": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "b200_linear_rms_input": (c_int, [c_void_p] * 5 + [c_int64] * 5 + [c_double, c_int, c_void_p,
                                                                       c_void_p]),
    "b200_linear_splitk_slices": (c_int64, [c_int64] * 3),
    "b200_linear_splitk_residual": (c_int, [c_void_p] * 5 + [c_int64] * 4 + [c_void_p, c_void_p]),
    "b200_embedding": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int,
                               c_void_p, c_void_p]),
    "b200_swiglu": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "b200_add": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "b200_copy_4d": (c_int, [c_void_p, c_void_p, _I64P, _I64P, c_int, c_int, c_void_p]),
    "b200_advance_lengths": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p,
                                     c_void_p]),
    "b200_argmax": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p]),
}

_library: ctypes.CDLL | None = None


def load() -> ctypes.CDLL:
    """Loads the library once and binds every declared symbol."""

    global _library
    if _library is not None:
        return _library
    if not LIBRARY_PATH.exists():
        raise B200LibraryError(
            f"{LIBRARY_PATH} not found: build it with `python {PACKAGE_DIR.name}/build.py` "
            "(there is no fallback path)"
        )
    library = ctypes.CDLL(str(LIBRARY_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        try:
            function = getattr(library, name)
        except AttributeError as error:
            raise B200LibraryError(f"{LIBRARY_PATH} does not export {name}") from error
        function.restype = restype
        function.argtypes = argtypes
    _library = library
    return library


def error_string(code: int) -> str:
    return load().b200_error_string(code).decode()


def i64_array(values) -> ctypes.Array:
    values = [int(v) for v in values]
    return (c_int64 * len(values))(*values)
