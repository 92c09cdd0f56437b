"""The C-ABI library loads on a machine without a GPU and exports exactly what
include/b200_serve.h declares; host-side argument checks reject bad requests before any
launch (no compute call is made here)."""

import ctypes
import re
from pathlib import Path

import pytest

from llm_compiler_b200 import _lib

HEADER = Path(__file__).resolve().parent.parent / "include" / "b200_serve.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(b200_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    names = declared_functions()
    assert len(names) >= 18
    library = _lib.load()
    for name in names:
        assert hasattr(library, name), f"{name} is declared but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names


def test_abi_version_and_error_strings():
    library = _lib.load()
    assert library.b200_abi_version() == _lib.ABI_VERSION == 104
    assert _lib.error_string(0) == "ok"
    for code in range(-6, 0):
        assert _lib.error_string(code) not in ("ok", "unknown error code")


def test_host_side_rejections_happen_before_any_launch():
    library = _lib.load()
    strides = _lib.i64_array([0, 0, 0, 1])
    # null pointers
    assert library.b200_kv_store(None, None, None, None, None, 1, 8, 2, 1, 64, strides, strides,
                                 _lib.BF16, None, None) == _lib.ERR_BAD_ARGUMENT
    assert library.b200_rms_norm(None, None, None, 1, 64, 64, 1e-6, 1, 1, 1, 1, 0, None) == \
        _lib.ERR_BAD_ARGUMENT
    # sizes the workspace queries understand without a device
    assert library.b200_decode_attention_workspace_bytes(64, 14, 2, 64, 4096, 512) == \
        65536 + (64 * 14 * 8 * 66 * 4 + 255) // 256 * 256  # counters + fp32 split partials
    assert library.b200_decode_attention_workspace_bytes(64, 14, 2, 64, 4096, 4096) == 0
    assert library.b200_linear_workspace_bytes(64, 4864, 896, _lib.BF16, 0) > 0
    assert library.b200_linear_workspace_bytes(64, 896, 151936, _lib.BF16, 0) == 0
    fake = ctypes.c_void_p(256)  # never dereferenced: rejected on the host
    assert library.b200_linear(fake, fake, None, None, fake, 4, 7, 8, 7, _lib.BF16, 0, None, 0,
                               None, None) == _lib.ERR_UNSUPPORTED  # K not a multiple of 8
    assert library.b200_linear(fake, fake, None, None, fake, 4, 8, 8, 8, _lib.BF16, 1, None, 0,
                               None, None) == _lib.ERR_BAD_ARGUMENT  # residual epilogue without residual
    assert library.b200_decode_attention(fake, fake, fake, fake, None, fake, 2, 5, 2, 64, 16, 16,
                                         320, 64, 0, 0, 0.125, _lib.BF16, 0, 0, 0, None, 0, None,
                                         None) == _lib.ERR_BAD_ARGUMENT  # 5 heads over 2 KV heads


def test_missing_library_is_an_error(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_library", None)
    monkeypatch.setattr(_lib, "LIBRARY_PATH", tmp_path / "libb200serve.so")
    with pytest.raises(_lib.B200LibraryError):
        _lib.load()


def test_operands_on_another_gpu_are_refused_before_any_launch(monkeypatch):
    """The C ABI launches on the current device with the current stream; tensors of another
    GPU must be rejected on the host (nothing is launched, no GPU is needed for the check)."""
    import torch

    from llm_compiler_b200 import kernels

    monkeypatch.setattr(torch.cuda, "current_device", lambda: 0)
    kernels._guard_current_device(torch.device("cuda", 0))
    kernels._guard_current_device(torch.device("cuda"))  # no index: the current device
    with pytest.raises(ValueError, match="current device is cuda:0"):
        kernels._guard_current_device(torch.device("cuda", 1))
