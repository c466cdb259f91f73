"""Torch-facing wrappers of the C-ABI kernels.

Each function validates what only the Python side can know (device, dtype, contiguity of
the innermost dimension), passes raw device pointers, element strides and torch's current
stream to the library, and returns torch tensors.  CUDA tensors only.
"""
from typing import Optional, Tuple

import torch

from . import _capi
from ._capi import BASED_BF16, BASED_F32, IMPL_AUTO, IMPL_SIMT, IMPL_TCGEN05  # noqa: F401

EXPANDED_DIM = 273
_IMPLS = {"auto": IMPL_AUTO, "simt": IMPL_SIMT, "tcgen05": IMPL_TCGEN05}


def _dt(t: torch.dtype) -> int:
    if t == torch.float32:
        return BASED_F32
    if t == torch.bfloat16:
        return BASED_BF16
    raise TypeError(f"unsupported dtype {t}: the kernels take float32 or bfloat16")


def _need_cuda(*ts):
    """Every op starts here: CUDA tensors only, and no autograd.  The kernels write into fresh buffers through
    raw pointers and register no backward, so under grad mode the result would silently be cut off from the
    graph (the projections before a mixer would get no gradient and nothing would say so)."""
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("based_b200 ops run on CUDA tensors only (there is no CPU path)")
    if torch.is_grad_enabled():
        for t in ts:
            if t is not None and t.requires_grad:
                raise RuntimeError(
                    "based_b200 kernels are inference-only (no backward): call them under torch.no_grad() or "
                    "torch.inference_mode(), or detach the inputs")


def check_status(reset: bool = True) -> int:
    """Read the tensor-core kernels' status word and raise if a bounded in-kernel wait ever expired (the results
    of that launch are then meaningless).  It synchronises the device, so call it where the caller synchronises
    anyway: after a generation loop, at the end of a timed region."""
    code = _capi.read_status(reset)
    if code != 0:
        raise _capi.BasedLibraryError(f"a bounded wait expired inside a tensor-core kernel (status 0x{code:x}); "
                                      "the outputs of that launch are not valid")
    return code


def _inner_contig(t, name):
    if t.stride(-1) != 1:
        raise ValueError(f"{name}: innermost stride must be 1")


def _stream():
    return torch.cuda.current_stream().cuda_stream


def linattn_prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, eps: float = 1e-12,
                    return_state: bool = True, state_dtype: Optional[torch.dtype] = None,
                    out: Optional[torch.Tensor] = None, impl: str = "auto",
                    kv_state: Optional[torch.Tensor] = None, k_state: Optional[torch.Tensor] = None,
                    nseg: Optional[int] = None, scratch: Optional[torch.Tensor] = None,
                    ) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
    """Causal Taylor linear attention over a whole sequence.

    q, k ``[B, H, L, 16]`` (raw), v ``[B, H, L, dv]``; any batch/head/seq strides (e.g. the
    transposed views LinearAttention.forward makes, linear_attention.py:127-129).
    Returns ``y`` as a ``[B, H, L, dv]`` view of a ``[B, L, H, dv]`` buffer (so the reference's
    ``'b h l d -> b l (h d)'`` rearrange is free), ``kv_state [B, H, 1, dv, 273]`` and
    ``k_state [B, H, 1, 1, 273]`` (linear_attention.py:220-222), or ``None`` for the states
    when ``return_state`` is false.  ``kv_state``/``k_state`` may be given to be filled in place.

    ``nseg`` splits the SEQUENCE into that many segments that run on different SMs (bf16, tensor-core
    kernel only): ``None`` lets the library choose (it splits only when ``B*H`` is below half the SM
    count and ``L >= 1024``), ``1`` never splits.  The split needs a workspace of
    ``based_linattn_prefill_scratch_bytes`` bytes; ``scratch`` (a CUDA uint8/float tensor at least that
    large) may be given to reuse one, else it is taken from torch's caching allocator.
    """
    _need_cuda(q, k, v)
    B, H, L, d = q.shape
    dv = v.shape[-1]
    if k.shape != q.shape or v.shape[:3] != q.shape[:3]:
        raise ValueError("q, k, v shapes disagree")
    if not (q.dtype == k.dtype == v.dtype):
        raise TypeError("q, k, v must share a dtype")
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _inner_contig(t, n)
    if out is None:
        out = torch.empty(B, L, H, dv, dtype=q.dtype, device=q.device).permute(0, 2, 1, 3)
    else:
        _inner_contig(out, "out")
    sdt = kv_state.dtype if kv_state is not None else (state_dtype or q.dtype)
    if return_state:
        if kv_state is None:
            kv_state = torch.empty(B, H, 1, dv, EXPANDED_DIM, dtype=sdt, device=q.device)
            k_state = torch.empty(B, H, 1, 1, EXPANDED_DIM, dtype=sdt, device=q.device)
        elif not (kv_state.is_contiguous() and k_state.is_contiguous()):
            raise ValueError("kv_state / k_state must be contiguous")
    if L == 0 or B == 0 or H == 0:  # empty tensors have no device pointer to pass
        if return_state:
            kv_state.zero_()
            k_state.zero_()
        return out, (kv_state if return_state else None), (k_state if return_state else None)
    lib = _capi.lib()
    can_split = q.dtype == torch.bfloat16 and dv <= 112 and impl in ("auto", "tcgen05")
    if nseg is not None and nseg > 1 and not can_split:
        raise ValueError("nseg > 1 needs bf16 inputs, dv <= 112 and the tensor-core kernel")
    with torch.cuda.device(q.device):
        if nseg is None:
            nseg = lib.based_linattn_prefill_segments(B, H, L) if can_split else 1
        if nseg > 1:
            need = lib.based_linattn_prefill_scratch_bytes(B, H, L, dv, nseg)
            if scratch is None:
                scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=q.device)
            elif scratch.device != q.device or not scratch.is_contiguous():
                raise ValueError("scratch must be a contiguous tensor on the inputs' device")
            code = lib.based_linattn_prefill_split(
                q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                kv_state.data_ptr() if return_state else None, k_state.data_ptr() if return_state else None,
                B, H, L, d, dv,
                _capi.strides(*q.stride()[:3]), _capi.strides(*k.stride()[:3]),
                _capi.strides(*v.stride()[:3]), _capi.strides(*out.stride()[:3]),
                _dt(sdt), float(eps), int(nseg), scratch.data_ptr(), scratch.numel() * scratch.element_size(),
                _stream())
            _capi.check(code, "based_linattn_prefill_split")
            return out, (kv_state if return_state else None), (k_state if return_state else None)
        code = lib.based_linattn_prefill(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
            kv_state.data_ptr() if return_state else None, k_state.data_ptr() if return_state else None,
            B, H, L, d, dv,
            _capi.strides(*q.stride()[:3]), _capi.strides(*k.stride()[:3]),
            _capi.strides(*v.stride()[:3]), _capi.strides(*out.stride()[:3]),
            _dt(q.dtype), _dt(sdt), float(eps), _IMPLS[impl], _stream())
    _capi.check(code, "based_linattn_prefill")
    return out, (kv_state if return_state else None), (k_state if return_state else None)


def linattn_decode(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kv_state: torch.Tensor,
                   k_state: torch.Tensor, *, eps: float = 1e-12, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One recurrent step; ``kv_state``/``k_state`` are updated IN PLACE.

    q, k ``[B, H, 1, 16]`` or ``[B, H, 16]`` (raw), v ``[B, H, 1, dv]`` or ``[B, H, dv]``;
    ``kv_state [B, H, 1, dv, 273]``, ``k_state [B, H, 1, 1, 273]`` (fp32 or bf16).
    Returns ``y [B, 1, H*dv]`` in ``q.dtype`` (the layout recurrent_forward hands to out_proj,
    linear_attention.py:251).
    """
    _need_cuda(q, k, v, kv_state, k_state)
    if q.dim() == 4:
        q, k, v = q[:, :, 0], k[:, :, 0], v[:, :, 0]
    B, H, d = q.shape
    dv = v.shape[-1]
    if kv_state.shape != (B, H, 1, dv, EXPANDED_DIM) or k_state.shape != (B, H, 1, 1, EXPANDED_DIM):
        raise ValueError(f"state shapes {tuple(kv_state.shape)}, {tuple(k_state.shape)} do not match B={B} H={H} dv={dv}")
    if not (kv_state.is_contiguous() and k_state.is_contiguous()):
        raise ValueError("kv_state / k_state must be contiguous")
    if kv_state.dtype != k_state.dtype:
        raise TypeError("kv_state and k_state must share a dtype")
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _inner_contig(t, n)
    if out is None:
        out = torch.empty(B, 1, H * dv, dtype=q.dtype, device=q.device)
    y = out.view(B, H, dv)
    with torch.cuda.device(q.device):
        code = _capi.lib().based_linattn_decode(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), y.data_ptr(), kv_state.data_ptr(), k_state.data_ptr(),
            B, H, d, dv, _capi.strides(*q.stride()[:2]), _capi.strides(*k.stride()[:2]),
            _capi.strides(*v.stride()[:2]), _capi.strides(*y.stride()[:2]),
            _dt(q.dtype), _dt(kv_state.dtype), float(eps), _stream())
    _capi.check(code, "based_linattn_decode")
    return out


def swa_prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window_left: int,
                softmax_scale: Optional[float] = None, *, impl: str = "auto",
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal sliding-window softmax attention; q, k, v ``[B, L, H, hd]`` (views into a packed
    qkv tensor are fine).  Query i sees keys ``[i - window_left, i]`` (slide_attention.py:97)."""
    _need_cuda(q, k, v)
    B, L, H, hd = q.shape
    if k.shape != q.shape or v.shape != q.shape:
        raise ValueError("q, k, v shapes disagree")
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _inner_contig(t, n)
    if out is None:
        out = torch.empty(B, L, H, hd, dtype=q.dtype, device=q.device)
    scale = hd ** -0.5 if softmax_scale is None else float(softmax_scale)
    if out.numel() == 0:
        return out
    with torch.cuda.device(q.device):
        code = _capi.lib().based_swa_prefill(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, L, H, hd,
            _capi.strides(*q.stride()[:3]), _capi.strides(*k.stride()[:3]),
            _capi.strides(*v.stride()[:3]), _capi.strides(*out.stride()[:3]),
            int(window_left), scale, _dt(q.dtype), _IMPLS[impl], _stream())
    _capi.check(code, "based_swa_prefill")
    return out


def swa_decode(q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, kv_cache: torch.Tensor,
               cache_seqlens, window_left: int, softmax_scale: Optional[float] = None, *,
               rotary_cos: Optional[torch.Tensor] = None, rotary_sin: Optional[torch.Tensor] = None,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One decode step: optional RoPE at the new position, append to ``kv_cache
    [B, maxL, 2, H, hd]`` IN PLACE, attend over the window (slide_attention.py:414-427).
    q, k_new, v_new ``[B, 1, H, hd]``; ``cache_seqlens`` an int or an int32 ``[B]`` CUDA tensor."""
    _need_cuda(q, k_new, v_new, kv_cache)
    B, one, H, hd = q.shape
    assert one == 1
    if not kv_cache.is_contiguous() or kv_cache.shape[0] < B or kv_cache.shape[2:] != (2, H, hd):
        raise ValueError("kv_cache must be contiguous [B, maxL, 2, H, hd]")
    if kv_cache.dtype != q.dtype:
        raise TypeError("kv_cache and q must share a dtype")
    q3, k3, v3 = q[:, 0], k_new[:, 0], v_new[:, 0]
    for t, n in ((q3, "q"), (k3, "k_new"), (v3, "v_new")):
        _inner_contig(t, n)
    if out is None:
        out = torch.empty(B, 1, H, hd, dtype=q.dtype, device=q.device)
    o3 = out[:, 0]
    if torch.is_tensor(cache_seqlens):
        if cache_seqlens.dtype != torch.int32 or not cache_seqlens.is_cuda or not cache_seqlens.is_contiguous():
            raise TypeError("cache_seqlens must be a contiguous int32 CUDA tensor")
        import ctypes
        lens_ptr = ctypes.cast(cache_seqlens.data_ptr(), ctypes.POINTER(ctypes.c_int32))
        lens_scalar = 0
    else:
        lens_ptr, lens_scalar = None, int(cache_seqlens)
    rdim = 0
    if rotary_cos is not None:
        if rotary_cos.dtype != q.dtype or rotary_sin.dtype != q.dtype:
            raise TypeError("rotary tables must be in the q dtype")
        if not (rotary_cos.is_contiguous() and rotary_sin.is_contiguous()):
            raise ValueError("rotary tables must be contiguous")
        rdim = 2 * rotary_cos.shape[-1]
    scale = hd ** -0.5 if softmax_scale is None else float(softmax_scale)
    with torch.cuda.device(q.device):
        code = _capi.lib().based_swa_decode(
            q3.data_ptr(), k3.data_ptr(), v3.data_ptr(), o3.data_ptr(), kv_cache.data_ptr(), lens_ptr, lens_scalar,
            rotary_cos.data_ptr() if rotary_cos is not None else None,
            rotary_sin.data_ptr() if rotary_sin is not None else None, rdim,
            B, H, hd, kv_cache.shape[1], _capi.strides(*q3.stride()[:2]), _capi.strides(*k3.stride()[:2]),
            _capi.strides(*v3.stride()[:2]), _capi.strides(*o3.stride()[:2]),
            int(window_left), scale, _dt(q.dtype), _stream())
    _capi.check(code, "based_swa_decode")
    return out


def rotary_apply_(x: torch.Tensor, rotary_cos: torch.Tensor, rotary_sin: torch.Tensor, seqlen_offset=0) -> torch.Tensor:
    """In-place non-interleaved RoPE on ``x [B, L, H, hd]`` (a view into packed qkv is fine);
    ``seqlen_offset`` an int or an int32 ``[B]`` CUDA tensor (based/ops/triton/rotary.py:68-105)."""
    _need_cuda(x, rotary_cos, rotary_sin)
    B, L, H, hd = x.shape
    _inner_contig(x, "x")
    if rotary_cos.dtype != x.dtype or rotary_sin.dtype != x.dtype:
        raise TypeError("rotary tables must be in the dtype of x")
    if not (rotary_cos.is_contiguous() and rotary_sin.is_contiguous()):
        raise ValueError("rotary tables must be contiguous")
    if x.numel() == 0:
        return x
    if torch.is_tensor(seqlen_offset):
        import ctypes
        if seqlen_offset.dtype != torch.int32 or not seqlen_offset.is_cuda:
            raise TypeError("seqlen_offset tensor must be int32 on CUDA")
        off_ptr, off_scalar = ctypes.cast(seqlen_offset.data_ptr(), ctypes.POINTER(ctypes.c_int32)), 0
        max_pos = None
    else:
        off_ptr, off_scalar = None, int(seqlen_offset)
        if off_scalar + L > rotary_cos.shape[0]:
            raise ValueError("rotary tables are shorter than seqlen_offset + L")
    with torch.cuda.device(x.device):
        code = _capi.lib().based_rotary_apply(
            x.data_ptr(), B, L, H, hd, _capi.strides(*x.stride()[:3]), rotary_cos.data_ptr(), rotary_sin.data_ptr(),
            2 * rotary_cos.shape[-1], off_ptr, off_scalar, _dt(x.dtype), _stream())
    _capi.check(code, "based_rotary_apply")
    return x


def gated_conv_prefill(u: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, *,
                       state: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``silu(causal_depthwise_conv(u1) + bias) * u2`` with ``u1, u2`` the halves of ``u [B, L, 2*di]``.

    ``weight [di, k]`` (or ``[di, 1, k]`` as nn.Conv1d stores it), ``bias [di]`` or None, both in one
    dtype (float32 or bfloat16).  ``state [B, di, k]`` (dtype of ``u``), when given, receives the
    last k inputs of the convolution (convolution.py:63-67).  Returns ``v [B, L, di]``.
    """
    _need_cuda(u, weight, bias, state)
    B, L, two_di = u.shape
    di = two_di // 2
    weight = weight.reshape(weight.shape[0], -1)
    k = weight.shape[1]
    if weight.shape[0] != di or two_di != 2 * di:
        raise ValueError("u must be [B, L, 2*di] and weight [di, k]")
    _inner_contig(u, "u")
    weight = weight.contiguous()
    if bias is not None:
        bias = bias.to(weight.dtype).contiguous()
    if out is None:
        out = torch.empty(B, L, di, dtype=u.dtype, device=u.device)
    else:
        _inner_contig(out, "out")
    if state is not None and (state.shape != (B, di, k) or state.dtype != u.dtype or not state.is_contiguous()):
        raise ValueError("state must be a contiguous [B, di, k] tensor of u's dtype")
    if B == 0 or L == 0:
        if state is not None:
            state.zero_()
        return out
    u1, u2 = u[..., :di], u[..., di:]
    with torch.cuda.device(u.device):
        code = _capi.lib().based_gated_conv_prefill(
            u1.data_ptr(), u2.data_ptr(), out.data_ptr(), state.data_ptr() if state is not None else None,
            weight.data_ptr(), bias.data_ptr() if bias is not None else None, B, L, di, k,
            _capi.strides(*u1.stride()[:2]), _capi.strides(*u2.stride()[:2]), _capi.strides(*out.stride()[:2]),
            _dt(u.dtype), _dt(weight.dtype), _stream())
    _capi.check(code, "based_gated_conv_prefill")
    return out


def gated_conv_step(u: torch.Tensor, state: torch.Tensor, weight: torch.Tensor,
                    bias: Optional[torch.Tensor] = None, *, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One decode step of :func:`gated_conv_prefill`; ``state [B, di, k]`` is updated IN PLACE
    (convolution.py:104-107).  ``u [B, 2*di]`` or ``[B, 1, 2*di]``; returns ``[B, di]``."""
    _need_cuda(u, state, weight, bias)
    if u.dim() == 3:
        u = u[:, 0]
    B, two_di = u.shape
    di = two_di // 2
    weight = weight.reshape(weight.shape[0], -1).contiguous()
    k = weight.shape[1]
    _inner_contig(u, "u")
    if bias is not None:
        bias = bias.to(weight.dtype).contiguous()
    if state.shape != (B, di, k) or state.dtype != u.dtype or not state.is_contiguous():
        raise ValueError("state must be a contiguous [B, di, k] tensor of u's dtype")
    if out is None:
        out = torch.empty(B, di, dtype=u.dtype, device=u.device)
    if B == 0:
        return out
    u1, u2 = u[:, :di], u[:, di:]
    with torch.cuda.device(u.device):
        code = _capi.lib().based_gated_conv_step(
            u1.data_ptr(), u2.data_ptr(), out.data_ptr(), state.data_ptr(), weight.data_ptr(),
            bias.data_ptr() if bias is not None else None, B, di, k, u1.stride(0), u2.stride(0), out.stride(0),
            _dt(u.dtype), _dt(weight.dtype), _stream())
    _capi.check(code, "based_gated_conv_step")
    return out


def add_rmsnorm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                residual: Optional[torch.Tensor] = None, *, eps: float = 1e-6, prenorm: bool = False,
                residual_in_fp32: bool = False, round_input: bool = False):
    """``z = x + residual``; ``out = rmsnorm(z) * weight (+ bias)`` in one pass; with ``prenorm`` returns
    ``(out, z)`` like rms_norm_fn (layer_norm.py:926-953).  ``z`` is fp32 when ``residual_in_fp32`` or
    when ``residual`` already is, else x's dtype.  ``round_input`` rounds ``z`` to x's dtype before the
    norm (the unfused ``norm(residual.to(weight.dtype))`` of block.py:134-137).  x ``[..., D]``."""
    _need_cuda(x, weight, bias, residual)
    D = x.shape[-1]
    x2 = x.reshape(-1, D)
    _inner_contig(x2, "x")
    M = x2.shape[0]
    res2 = None
    if residual is not None:
        if residual.shape != x.shape:
            raise ValueError("residual must have x's shape")
        res2 = residual.reshape(-1, D)
        _inner_contig(res2, "residual")
    res_dtype = torch.float32 if (residual_in_fp32 or (residual is not None and residual.dtype == torch.float32)) else x.dtype
    if res2 is not None and res2.dtype != res_dtype:
        res2 = res2.to(res_dtype)
    weight = weight.contiguous()
    if bias is not None:
        bias = bias.to(weight.dtype).contiguous()
    out = torch.empty(M, D, dtype=x.dtype, device=x.device)
    res_out = torch.empty(M, D, dtype=res_dtype, device=x.device) if prenorm else None
    if M > 0:
        with torch.cuda.device(x.device):
            code = _capi.lib().based_add_rmsnorm(
                x2.data_ptr(), res2.data_ptr() if res2 is not None else None, weight.data_ptr(),
                bias.data_ptr() if bias is not None else None, out.data_ptr(),
                res_out.data_ptr() if res_out is not None else None, M, D, x2.stride(0),
                res2.stride(0) if res2 is not None else 0, out.stride(0), res_out.stride(0) if res_out is not None else 0,
                float(eps), _dt(x.dtype), _dt(res_dtype), _dt(weight.dtype), int(round_input), _stream())
        _capi.check(code, "based_add_rmsnorm")
    out = out.reshape(x.shape)
    return (out, res_out.reshape(x.shape)) if prenorm else out


_ACTS = {"silu": 0, "swiglu": 0, "sigmoid": 1, "glu": 1}


def gated_act(y: torch.Tensor, activation: str = "silu") -> torch.Tensor:
    """``first_half * act(second_half)`` over the last dim of ``y [..., 2F]`` (mlp.py:141-154)."""
    _need_cuda(y)
    F2 = y.shape[-1]
    F = F2 // 2
    y2 = y.reshape(-1, F2)
    _inner_contig(y2, "y")
    M = y2.shape[0]
    out = torch.empty(M, F, dtype=y.dtype, device=y.device)
    if M > 0:
        a, g = y2[:, :F], y2[:, F:]
        with torch.cuda.device(y.device):
            code = _capi.lib().based_gated_act(a.data_ptr(), g.data_ptr(), out.data_ptr(), M, F, a.stride(0),
                                               g.stride(0), out.stride(0), _ACTS[activation], _dt(y.dtype), _stream())
        _capi.check(code, "based_gated_act")
    return out.reshape(*y.shape[:-1], F)


DECODE_LINEAR_MAX_ROWS = 64  # beyond this the library GEMM is the better tool
# Which decode-step products the mixers and the MLP hand to decode_linear instead of cuBLAS (+ a separate
# elementwise launch).  Measured on the 360M model at batch 16 with the weights streaming from HBM
# (ms per decode step): none 1.146, gated 1.089, gated + conv 1.145, all three 1.329 -- only fc1 + SwiGLU pays.
DECODE_LINEAR_USE = {"plain": False, "gated": True, "conv": False}


def decode_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, *,
                  epilogue: str = "plain", activation: str = "silu", conv_state: Optional[torch.Tensor] = None,
                  conv_weight: Optional[torch.Tensor] = None, conv_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x W^T (+ bias)`` for the few rows of a decode step (bf16), with a fused epilogue:
    ``"plain"``; ``"gated"`` -> ``first_half * act(second_half)`` (mlp.py:146-154); ``"conv"`` -> the BaseConv
    decode step on the first half (``conv_state [M, N/2, k]`` updated in place), silu, gate by the second half
    (convolution.py:88-109, :205-211).  x ``[..., K]``; returns ``[..., N]`` or ``[..., N/2]``."""
    _need_cuda(x, weight, bias, conv_state, conv_weight, conv_bias)
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise TypeError("decode_linear takes bfloat16 activations and weights")
    K = x.shape[-1]
    x2 = x.reshape(-1, K)
    _inner_contig(x2, "x")
    M, N = x2.shape[0], weight.shape[0]
    if weight.shape[1] != K or not weight.is_contiguous():
        raise ValueError("weight must be a contiguous [N, K] tensor")
    epi = {"plain": 0, "gated": 1, "conv": 2}[epilogue]
    n_out = N if epi == 0 else N // 2
    out = torch.empty(M, n_out, dtype=torch.bfloat16, device=x.device)
    if bias is not None:
        bias = bias.to(torch.bfloat16).contiguous()
    ck, cw_dt = 0, BASED_BF16
    if epi == 2:
        conv_weight = conv_weight.reshape(conv_weight.shape[0], -1).contiguous()
        ck, cw_dt = conv_weight.shape[1], _dt(conv_weight.dtype)
        if conv_bias is not None:
            conv_bias = conv_bias.to(conv_weight.dtype).contiguous()
        if conv_state.shape != (M, n_out, ck) or conv_state.dtype != torch.bfloat16 or not conv_state.is_contiguous():
            raise ValueError("conv_state must be a contiguous bfloat16 [M, N/2, k] tensor")
    if M > 0:
        with torch.cuda.device(x.device):
            code = _capi.lib().based_decode_linear(
                x2.data_ptr(), weight.data_ptr(), bias.data_ptr() if bias is not None else None, out.data_ptr(),
                M, N, K, x2.stride(0), out.stride(0), epi, _ACTS[activation],
                conv_state.data_ptr() if epi == 2 else None, conv_weight.data_ptr() if epi == 2 else None,
                conv_bias.data_ptr() if (epi == 2 and conv_bias is not None) else None, ck, cw_dt, _stream())
        _capi.check(code, "based_decode_linear")
    return out.reshape(*x.shape[:-1], n_out)


def _decode_rows(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """True when ``x W^T`` is a decode-step product the library's own kernel should run."""
    rows = x.numel() // x.shape[-1] if x.numel() else 0
    return (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and 0 < rows <= DECODE_LINEAR_MAX_ROWS
            and x.shape[-1] % 32 == 0 and weight.shape[0] % 8 == 0 and weight.is_contiguous() and x.stride(-1) == 1
            and not torch.is_grad_enabled())


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``nn.functional.linear`` for the mixers: the decode-step kernel for a few bf16 rows, cuBLAS otherwise."""
    if DECODE_LINEAR_USE["plain"] and _decode_rows(x, weight):
        return decode_linear(x, weight, bias)
    return torch.nn.functional.linear(x, weight, bias)


def rotary_qkv_cache_(qkv: torch.Tensor, rotary_cos: torch.Tensor, rotary_sin: torch.Tensor,
                      kv_cache: torch.Tensor) -> torch.Tensor:
    """Prompt pass of the sliding-window mixer: whole-head RoPE on q and k of packed ``qkv [B, L, 3, H, hd]`` in
    place, and rotated k plus v written to ``kv_cache[:B, :L]`` (``[*, max_seqlen, 2, H, hd]``) in the same launch
    (slide_attention.py:553-556 and :255-281).  bf16 only; returns ``qkv``."""
    _need_cuda(qkv, rotary_cos, rotary_sin, kv_cache)
    B, L, three, H, hd = qkv.shape
    if three != 3 or qkv.dtype != torch.bfloat16 or kv_cache.dtype != torch.bfloat16:
        raise TypeError("rotary_qkv_cache_ takes a bfloat16 [B, L, 3, H, hd] tensor and a bfloat16 cache")
    _inner_contig(qkv, "qkv")
    if rotary_cos.shape[-1] * 2 != hd or rotary_cos.shape[0] < L or rotary_cos.dtype != torch.bfloat16:
        raise ValueError("rotary tables must be bfloat16 [>= L, hd/2]")
    if not (rotary_cos.is_contiguous() and rotary_sin.is_contiguous()):
        raise ValueError("rotary tables must be contiguous")
    if (kv_cache.shape[0] < B or kv_cache.shape[1] < L or tuple(kv_cache.shape[2:]) != (2, H, hd)
            or kv_cache.stride()[2:] != (H * hd, hd, 1)):
        raise ValueError("kv_cache must be [>= B, >= L, 2, H, hd] with the last three dims contiguous")
    if qkv.numel() == 0:
        return qkv
    with torch.cuda.device(qkv.device):
        code = _capi.lib().based_rotary_qkv_cache(
            qkv.data_ptr(), B, L, H, hd, _capi.strides(*qkv.stride()[:4]), rotary_cos.data_ptr(), rotary_sin.data_ptr(),
            kv_cache.data_ptr(), _capi.strides(*kv_cache.stride()[:2]), _stream())
    _capi.check(code, "based_rotary_qkv_cache")
    return qkv


def tp_outproj_workspace_bytes(world: int, max_rows: int, n_out: int) -> int:
    """Size of one rank's receive workspace for :func:`tp_outproj_allreduce`."""
    n = _capi.lib().based_tp_outproj_workspace_bytes(int(world), int(max_rows), int(n_out))
    if n == 0:
        raise ValueError("tp_outproj: world must be 1..8, max_rows >= 1 and n_out a multiple of 8")
    return n


def tp_outproj_workspace_init_(ws: torch.Tensor) -> torch.Tensor:
    """Prepare a workspace (zero flags, call counter = 1).  Once, by its owner, before any rank's first call."""
    _need_cuda(ws)
    with torch.cuda.device(ws.device):
        _capi.check(_capi.lib().based_tp_outproj_workspace_init(ws.data_ptr(), ws.numel() * ws.element_size(), _stream()),
                    "based_tp_outproj_workspace_init")
    return ws


def tp_outproj_allreduce(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], workspace_ptrs, max_rows: int,
                         rank: int, world: int, *, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row-parallel ``x W^T`` summed over the tensor-parallel ranks (+ bias), one kernel per rank
    (based/ops/fused_dense.py:239-246 as GEMM + all-reduce in one launch).  ``x [..., K_local]`` bf16 with at most
    ``max_rows`` rows, ``weight [N, K_local]`` bf16 contiguous; ``workspace_ptrs`` the device addresses of every rank's
    workspace as mapped in this process.  A collective: every rank calls it with the same shapes."""
    _need_cuda(x, weight, bias)
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise TypeError("tp_outproj_allreduce takes bfloat16 activations and weights")
    K = x.shape[-1]
    x2 = x.reshape(-1, K)
    _inner_contig(x2, "x")
    M, N = x2.shape[0], weight.shape[0]
    if weight.shape[1] != K or not weight.is_contiguous():
        raise ValueError("weight must be a contiguous [N, K] tensor")
    if not 0 < M <= max_rows:
        raise ValueError(f"tp_outproj_allreduce: {M} rows, workspace built for at most {max_rows}")
    if len(workspace_ptrs) != world:
        raise ValueError("one workspace address per rank is needed")
    if bias is not None:
        bias = bias.to(torch.bfloat16).contiguous()
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    o2 = out.reshape(-1, N)
    with torch.cuda.device(x.device):
        code = _capi.lib().based_tp_outproj_allreduce(
            x2.data_ptr(), weight.data_ptr(), bias.data_ptr() if bias is not None else None, o2.data_ptr(), M, N, K,
            x2.stride(0), o2.stride(0), _capi.pointers(workspace_ptrs), int(max_rows), int(rank), int(world), _stream())
    _capi.check(code, "based_tp_outproj_allreduce")
    return out.reshape(*x.shape[:-1], N)


def tp_outproj_allreduce_emulated(xs, weights, bias, workspaces, max_rows: int):
    """All ranks of :func:`tp_outproj_allreduce` inside one cooperative launch on one GPU: ``xs[r] [M, K]``,
    ``weights[r] [N, K]``, ``workspaces[r]`` (prepared uint8 tensors), all on the same device.  Returns the list of the
    ranks' outputs.  For checking the exchange protocol with a single GPU."""
    world = len(xs)
    _need_cuda(*xs, *weights, bias, *workspaces)
    M, K = xs[0].shape
    N = weights[0].shape[0]
    outs = [torch.empty(M, N, dtype=torch.bfloat16, device=xs[0].device) for _ in range(world)]
    if bias is not None:
        bias = bias.to(torch.bfloat16).contiguous()
    with torch.cuda.device(xs[0].device):
        code = _capi.lib().based_tp_outproj_allreduce_emulated(
            _capi.pointers([t.data_ptr() for t in xs]), _capi.pointers([t.data_ptr() for t in weights]),
            bias.data_ptr() if bias is not None else None, _capi.pointers([t.data_ptr() for t in outs]), M, N, K,
            xs[0].stride(0), outs[0].stride(0), _capi.pointers([t.data_ptr() for t in workspaces]), int(max_rows), world,
            _stream())
    _capi.check(code, "based_tp_outproj_allreduce_emulated")
    return outs
