"""The C-ABI library: it loads, exports every symbol the header declares, and rejects bad
arguments on the host (no GPU needed: validation happens before any CUDA call)."""
import ctypes
import os
import re

import pytest

from conftest import ROOT
from based_b200 import _capi, build_library


@pytest.fixture(scope="module")
def lib():
    build_library()
    return _capi.lib()


def test_header_symbols_exported(lib):
    header = open(os.path.join(ROOT, "include", "based_b200.h")).read()
    declared = set(re.findall(r"\b(based_[a-z0-9_]+)\s*\(", header))
    assert declared == set(_capi.SIGNATURES), (declared, set(_capi.SIGNATURES))
    for name in declared:
        assert hasattr(lib, name)
    assert lib.based_b200_version() >= 1


def test_error_strings(lib):
    assert lib.based_error_string(0) == b"ok"
    for code in (-1, -2, -3, -4, -5, -6):
        assert lib.based_error_string(code) not in (b"ok", b"unknown error")


def test_prefill_rejects_bad_arguments(lib):
    s3 = _capi.strides(1, 1, 1)
    p = ctypes.c_void_p(256)  # never dereferenced: validation fails first
    f = lib.based_linattn_prefill
    assert f(None, p, p, p, None, None, 1, 1, 8, 16, 64, s3, s3, s3, s3, 0, 0, 1e-12, 0, None) == -1
    assert f(p, p, p, p, p, None, 1, 1, 8, 16, 64, s3, s3, s3, s3, 0, 0, 1e-12, 0, None) == -1
    assert f(p, p, p, p, None, None, 1, 1, 8, 8, 64, s3, s3, s3, s3, 0, 0, 1e-12, 0, None) == -2   # d != 16
    assert f(p, p, p, p, None, None, 1, 1, 8, 16, 72, s3, s3, s3, s3, 0, 0, 1e-12, 0, None) == -2  # dv % 16
    assert f(p, p, p, p, None, None, 1, 1, 8, 16, 64, s3, s3, s3, s3, 7, 0, 1e-12, 0, None) == -3
    assert f(p, p, p, p, None, None, 1, 1, 8, 16, 64, s3, s3, s3, s3, 0, 0, 1e-12, 2, None) == -5  # tcgen05 on fp32
    assert f(p, p, p, p, None, None, 0, 1, 8, 16, 64, s3, s3, s3, s3, 0, 0, 1e-12, 0, None) == 0   # empty batch


def test_decode_rejects_bad_arguments(lib):
    s2 = _capi.strides(1, 1)
    p = ctypes.c_void_p(256)
    f = lib.based_linattn_decode
    assert f(p, p, p, p, None, p, 1, 1, 16, 64, s2, s2, s2, s2, 1, 0, 1e-12, None) == -1
    assert f(p, p, p, p, p, p, 1, 1, 16, 200, s2, s2, s2, s2, 1, 0, 1e-12, None) == -2
    assert f(p, p, p, p, ctypes.c_void_p(260), p, 1, 1, 16, 64, s2, s2, s2, s2, 1, 0, 1e-12, None) == -4
    assert f(p, p, p, p, p, p, 1, 1, 16, 64, s2, s2, s2, s2, 1, 5, 1e-12, None) == -3


def test_swa_rejects_bad_arguments(lib):
    s3, s2 = _capi.strides(1, 1, 1), _capi.strides(1, 1)
    p = ctypes.c_void_p(256)
    assert lib.based_swa_prefill(p, p, p, None, 1, 8, 1, 64, s3, s3, s3, s3, 64, 0.125, 1, 0, None) == -1
    assert lib.based_swa_prefill(p, p, p, p, 1, 8, 1, 60, s3, s3, s3, s3, 64, 0.125, 1, 0, None) == -2
    assert lib.based_swa_prefill(p, p, p, p, 1, 8, 1, 64, s3, s3, s3, s3, -1, 0.125, 1, 0, None) == -2
    g = lib.based_swa_decode
    assert g(p, p, p, p, p, None, 9, None, None, 0, 1, 1, 64, 8, s2, s2, s2, s2, 64, 0.125, 1, None) == -2  # pos >= maxL
    assert g(p, p, p, p, p, None, 0, p, None, 64, 1, 1, 64, 8, s2, s2, s2, s2, 64, 0.125, 1, None) == -1    # cos w/o sin


def test_ops_refuse_cpu_tensors():
    import torch
    from based_b200 import ops
    q = torch.zeros(1, 1, 4, 16)
    with pytest.raises(RuntimeError):
        ops.linattn_prefill(q, q, torch.zeros(1, 1, 4, 64))


def test_split_prefill_plan_and_rejections(lib):
    """Segment planning is host arithmetic; the workspace size follows the segment count actually used."""
    f = lib.based_linattn_prefill_scratch_bytes
    assert f(1, 16, 32768, 64, 1) == 0
    # 256 chunks in 9 requested segments -> 29 chunks per segment -> 9 segments -> 8 stored states
    assert f(1, 16, 32768, 64, 9) == 16 * 8 * 65 * 160 * 4
    # more segments than chunks: one chunk per segment
    assert f(1, 1, 300, 64, 64) == 1 * 2 * 65 * 160 * 4
    s3 = _capi.strides(8, 8, 8)
    p = ctypes.c_void_p(256)
    g = lib.based_linattn_prefill_split
    assert g(p, p, p, p, None, None, 1, 1, 256, 16, 64, s3, s3, s3, s3, 0, 1e-12, 0, None, 0, None) == -2   # nseg < 1
    assert g(None, p, p, p, None, None, 1, 1, 256, 16, 64, s3, s3, s3, s3, 0, 1e-12, 2, None, 0, None) == -1
    assert g(p, p, p, p, None, None, 0, 1, 256, 16, 64, s3, s3, s3, s3, 0, 1e-12, 2, None, 0, None) == 0    # empty batch
    h = lib.based_linattn_prefill_split_static
    assert h(p, p, p, p, None, None, 1, 1, 256, 16, 64, s3, s3, s3, s3, 0, 1e-12, 0, None) == -2


def test_block_level_entry_points_reject_bad_arguments(lib):
    p = ctypes.c_void_p(256)
    s2 = _capi.strides(64, 64)
    conv = lib.based_gated_conv_prefill
    assert conv(None, p, p, None, p, None, 1, 4, 64, 3, s2, s2, s2, 1, 1, None) == -1
    assert conv(p, p, p, None, p, None, 1, 4, 64, 5, s2, s2, s2, 1, 1, None) == -2        # kernel size beyond 4
    assert conv(p, p, p, None, p, None, 1, 4, 64, 3, s2, s2, s2, 9, 1, None) == -3
    assert conv(p, p, p, None, p, None, 0, 4, 64, 3, s2, s2, s2, 1, 1, None) == 0
    step = lib.based_gated_conv_step
    assert step(p, p, p, None, p, None, 1, 64, 3, 64, 64, 64, 1, 1, None) == -1           # the state is required
    norm = lib.based_add_rmsnorm
    assert norm(p, None, None, None, p, None, 4, 64, 64, 0, 64, 0, 1e-5, 1, 0, 1, 0, None) == -1
    assert norm(p, None, p, None, p, None, 4, 0, 64, 0, 64, 0, 1e-5, 1, 0, 1, 0, None) == -2
    assert norm(p, None, p, None, p, None, 0, 64, 64, 0, 64, 0, 1e-5, 1, 0, 1, 0, None) == 0
    act = lib.based_gated_act
    assert act(p, p, p, 4, 64, 128, 128, 64, 7, 1, None) == -2                            # unknown activation
    assert act(p, None, p, 4, 64, 128, 128, 64, 0, 1, None) == -1
    lin = lib.based_decode_linear
    assert lin(p, p, None, p, 4, 64, 64, 64, 64, 2, 0, None, None, None, 3, 1, None) == -1  # conv epilogue needs a state
    assert lin(p, p, None, p, 4, 64, 64, 64, 64, 1, 9, None, None, None, 0, 1, None) == -2  # unknown activation
    assert lin(p, p, None, p, 0, 64, 64, 64, 64, 0, 0, None, None, None, 0, 1, None) == 0
    s4 = _capi.strides(8, 8, 8, 8)
    assert lib.based_rotary_qkv_cache(p, 1, 4, 2, 64, s4, p, p, None, s2, None) == -1
