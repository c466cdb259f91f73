"""The allocation-free sequence-split prefill (workspace built into the library) against the
entry point that takes the caller's workspace: bit-identical results on two calls in a row,
the capacity check, and no change in the device's free memory.  Collected last by name."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

STATIC_BYTES = 8 * 1024 * 1024


def _inputs(B, H, L, dv, seed):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, H, L, 16, generator=g) * 0.5).bfloat16().cuda()
    k = (torch.randn(B, H, L, 16, generator=g) * 0.5).bfloat16().cuda()
    v = torch.randn(B, H, L, dv, generator=g).bfloat16().cuda()
    return q, k, v


def _call_static(q, k, v, nseg):
    from based_b200 import _capi
    B, H, L, d = q.shape
    dv = v.shape[-1]
    y = torch.empty(B, H, L, dv, dtype=torch.bfloat16, device="cuda")
    kv = torch.empty(B, H, 1, dv, 273, dtype=torch.float32, device="cuda")
    ks = torch.empty(B, H, 1, 1, 273, dtype=torch.float32, device="cuda")
    code = _capi.lib().based_linattn_prefill_split_static(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), y.data_ptr(), kv.data_ptr(), ks.data_ptr(),
        B, H, L, d, dv,
        _capi.strides(*q.stride()[:3]), _capi.strides(*k.stride()[:3]),
        _capi.strides(*v.stride()[:3]), _capi.strides(*y.stride()[:3]),
        _capi.BASED_F32, ctypes.c_float(1e-12), nseg, torch.cuda.current_stream().cuda_stream)
    return code, y, kv, ks


def test_static_workspace_matches_caller_workspace_twice_in_a_row():
    from based_b200 import _capi, ops
    # two different problems back to back: the second finds the first one's leftovers in the array
    for seed, (B, H, L, dv, nseg) in enumerate([(1, 3, 4096 + 50, 64, 8), (2, 1, 2048, 112, 4)]):
        q, k, v = _inputs(B, H, L, dv, seed)
        code, y, kv, ks = _call_static(q, k, v, nseg)
        assert code == 0, _capi.lib().based_error_string(code)
        y_ref, kv_ref, ks_ref = ops.linattn_prefill(q, k, v, state_dtype=torch.float32, nseg=nseg)
        torch.cuda.synchronize()
        assert torch.equal(y, y_ref) and torch.equal(kv, kv_ref) and torch.equal(ks, ks_ref)
    # the same problem twice: identical results, and the device's free memory does not move
    q, k, v = _inputs(1, 2, 8192, 64, 7)
    code, y0, kv0, _ = _call_static(q, k, v, 16)
    torch.cuda.synchronize()
    assert code == 0
    free_before = torch.cuda.mem_get_info()[0]
    y = torch.empty_like(y0)
    kv = torch.empty_like(kv0)
    ks = torch.empty(1, 2, 1, 1, 273, dtype=torch.float32, device="cuda")
    lib = _capi.lib()
    for _ in range(2):
        code = lib.based_linattn_prefill_split_static(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), y.data_ptr(), kv.data_ptr(), ks.data_ptr(),
            1, 2, 8192, 16, 64,
            _capi.strides(*q.stride()[:3]), _capi.strides(*k.stride()[:3]),
            _capi.strides(*v.stride()[:3]), _capi.strides(*y.stride()[:3]),
            _capi.BASED_F32, ctypes.c_float(1e-12), 16, torch.cuda.current_stream().cuda_stream)
        assert code == 0
        torch.cuda.synchronize()
        assert torch.equal(y, y0) and torch.equal(kv, kv0)
    assert torch.cuda.mem_get_info()[0] == free_before
    assert _capi.read_status() == 0


def test_static_workspace_rejects_what_does_not_fit():
    from based_b200 import _capi
    lib = _capi.lib()
    B, H, L, dv, nseg = 1, 16, 4096, 64, 16       # 16 x 15 slots of 65 x 160 floats = 9.98 MB
    assert lib.based_linattn_prefill_scratch_bytes(B, H, L, dv, nseg) > STATIC_BYTES
    q, k, v = _inputs(B, H, L, dv, 3)
    code, _, _, _ = _call_static(q, k, v, nseg)
    assert code == -6                              # BASED_ERR_TOO_LARGE, nothing launched
    assert lib.based_linattn_prefill_scratch_bytes(B, H, L, dv, 8) <= STATIC_BYTES
    code, y, kv, _ = _call_static(q, k, v, 8)
    assert code == 0
    torch.cuda.synchronize()
    assert _capi.read_status() == 0
