"""CPU restatement of the Based hot path (TEST INFRASTRUCTURE, not product code).

Every function cites the file:line of HazyResearch/based it restates.  The
linear-attention functions are pinned against the reference's own PyTorch
modules: ``tests/golden/make_golden.py`` imports the reference, runs it on
seeded inputs and stores the results under ``tests/golden/``; the CPU tests
compare this file with those stored results.

The sliding-window functions restate the semantics of the reference's call
sites into flash-attn (pinned ``flash-attn==2.5.2`` in the reference's root
``setup.py:34``; its source is an un-vendored submodule and is not part of the
reference tree).  The reference has no CPU implementation of that mixer, so
those functions are pinned through ``tests/golden/swa_flash.npz``: outputs of
the flash-attn build installed in the image (2.8.3) called on a B200 with the
reference's own arguments by ``tests/golden/make_swa_golden_gpu.py`` (windowed
prefill at head_dim 64 / 112 and window 64 / 128; rotary + cache-append decode).

All functions run on CPU tensors in the dtype they are given (float64 and
float32 are the intended ones) and never touch CUDA.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch


# --------------------------------------------------------------------------
# TaylorExp feature map
# --------------------------------------------------------------------------
def taylor_exp(x: torch.Tensor) -> torch.Tensor:
    """2nd-order Taylor feature map, ``[..., d] -> [..., 1 + d + d*d]``.

    Restates ``TaylorExp.forward`` (based/models/mixers/linear_attention.py:67-75)
    with the constants of ``TaylorExp.__init__`` (:62-64): the second-order
    block holds all ``d*d`` products in row-major ``(i*d + j)`` order divided by
    ``sqrt(2)*sqrt(d)``; the first-order block is ``x / d**0.25``; the constant
    is 1.
    """
    d = x.shape[-1]
    r2 = math.sqrt(2.0)
    rd = math.sqrt(d)
    rrd = math.sqrt(rd)
    x2 = (x.unsqueeze(-1) * x.unsqueeze(-2)).flatten(start_dim=-2) / r2
    return torch.cat([torch.ones_like(x[..., :1]), x / rrd, x2 / rd], dim=-1)


def expanded_size(feature_dim: int) -> int:
    """``LinearAttention.expanded_size`` (linear_attention.py:255-256)."""
    return feature_dim * feature_dim + feature_dim + 1


# --------------------------------------------------------------------------
# LinearAttention: prefill (quadratic), state hand-off, recurrent step
# --------------------------------------------------------------------------
def linattn_parallel(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, eps: float = 1e-12
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Causal linear attention, quadratic form.

    q, k: ``[B, H, L, d]``; v: ``[B, H, L, dv]``.
    Returns ``y [B, H, L, dv]`` (before the ``b h l d -> b l (h d)`` rearrange
    and ``out_proj``), ``kv_state [B, H, 1, dv, D]`` and
    ``k_state [B, H, 1, 1, D]``.

    Restates the ``"quadratic"`` branch of ``LinearAttention.parallel_forward``
    (linear_attention.py:171-182) and the state hand-off (:220-222).
    """
    fq, fk = taylor_exp(q), taylor_exp(k)
    a = torch.einsum("bhnd,bhmd->bhnm", fq, fk)
    a = torch.tril(a)
    y = torch.einsum("bhnm,bhme->bhne", a, v)
    z = 1.0 / (torch.einsum("bhld,bhld->bhl", fq, fk.cumsum(2)) + eps)
    y = y * z[..., None]
    kv_state = torch.einsum("bhnd,bhnf->bhfd", fk, v)[:, :, None]
    k_state = fk.sum(dim=2)[:, :, None, None]
    return y, kv_state, k_state


def linattn_chunked(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    eps: float = 1e-12,
    chunk: int = 256,
    kv_state: Optional[torch.Tensor] = None,
    k_state: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Same results as :func:`linattn_parallel` in O(L) memory.

    The quadratic reference needs ``B*H*L*L`` elements; this evaluates it chunk
    by chunk, carrying ``kv_state``/``k_state`` in the reference layout between
    chunks (the identity the reference itself relies on: the recurrent state
    of linear_attention.py:240-241 summed over a chunk).  Used for long
    sequences after being checked against :func:`linattn_parallel` on short
    ones.
    """
    B, H, L, d = q.shape
    dv = v.shape[-1]
    D = expanded_size(d)
    if kv_state is None:
        kv_state = torch.zeros(B, H, 1, dv, D, dtype=q.dtype)
        k_state = torch.zeros(B, H, 1, 1, D, dtype=q.dtype)
    else:
        kv_state, k_state = kv_state.clone(), k_state.clone()
    ys = []
    for s in range(0, L, chunk):
        e = min(L, s + chunk)
        fq, fk = taylor_exp(q[:, :, s:e]), taylor_exp(k[:, :, s:e])
        vc = v[:, :, s:e]
        a = torch.tril(torch.einsum("bhnd,bhmd->bhnm", fq, fk))
        num = torch.einsum("bhnm,bhme->bhne", a, vc)
        num = num + torch.einsum("bhnf,bhef->bhne", fq, kv_state[:, :, 0])
        den = a.sum(-1) + torch.einsum("bhnf,bhf->bhn", fq, k_state[:, :, 0, 0])
        ys.append(num / (den + eps)[..., None])
        kv_state = kv_state + torch.einsum("bhnf,bhne->bhef", fk, vc)[:, :, None]
        k_state = k_state + fk.sum(2)[:, :, None, None]
    return torch.cat(ys, dim=2), kv_state, k_state


def linattn_recurrent_step(
    kv_state: torch.Tensor,
    k_state: torch.Tensor,
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    eps: float = 1e-12,
) -> torch.Tensor:
    """One decode step; updates ``kv_state``/``k_state`` IN PLACE.

    q, k: ``[B, H, 1, d]`` (raw, before the feature map); v: ``[B, H, 1, dv]``;
    ``kv_state [B, H, 1, dv, D]``; ``k_state [B, H, 1, 1, D]``.  Returns
    ``y [B, H, 1, dv]``.

    Restates the decode branch of ``LinearAttention.forward``
    (linear_attention.py:138-140, feature map applied first) and
    ``recurrent_forward`` (:230-251): state update first, readout second,
    denominator ``+ eps``.
    """
    fq, fk = taylor_exp(q), taylor_exp(k)
    fq_, fk_, v_ = fq.unsqueeze(-2), fk.unsqueeze(-2), v.unsqueeze(-1)
    kv_state += fk_[:, :, -1:] * v_[:, :, -1:]
    k_state += fk_[:, :, -1:]
    num = (fq_ * kv_state).sum(dim=-1)
    y = num / ((fq_ * k_state).sum(dim=-1) + eps)
    return y


def linattn_mixer_forward(
    x: torch.Tensor,
    wq: torch.Tensor,
    wk: torch.Tensor,
    wv: torch.Tensor,
    wo: torch.Tensor,
    num_heads: int,
    feature_dim: int,
    head_dim: int,
    eps: float = 1e-12,
):
    """Whole-mixer prefill: projections, attention, rearrange, ``out_proj``.

    Restates ``LinearAttention.forward`` (linear_attention.py:125-133) and the
    tail of ``parallel_forward`` (:183, :225).  Returns ``(out, kv_state,
    k_state)`` with ``out [B, L, d_model]``.
    """
    b, l, _ = x.shape
    q = (x @ wq.T).view(b, l, num_heads, feature_dim).transpose(1, 2)
    k = (x @ wk.T).view(b, l, num_heads, feature_dim).transpose(1, 2)
    v = (x @ wv.T).view(b, l, num_heads, head_dim).transpose(1, 2)
    y, kv_state, k_state = linattn_parallel(q, k, v, eps)
    y = y.transpose(1, 2).reshape(b, l, num_heads * head_dim)
    return y @ wo.T, kv_state, k_state


# --------------------------------------------------------------------------
# Rotary embedding (used by the sliding-window mixer in the full model)
# --------------------------------------------------------------------------
def rotary_cos_sin(seqlen: int, dim: int, base: float = 10000.0, dtype=torch.float32):
    """cos/sin tables ``[seqlen, dim/2]``.

    The reference builds them with flash-attn's ``RotaryEmbedding`` (call site
    based/models/mixers/slide_attention.py:349-355, :402-405); the published
    algorithm is ``inv_freq = base**(-arange(0, dim, 2)/dim)``,
    ``freqs = outer(arange(seqlen), inv_freq)`` in fp32, then cast to the
    model dtype.
    """
    inv_freq = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    t = torch.arange(seqlen, dtype=torch.float32)
    freqs = torch.outer(t, inv_freq)
    return torch.cos(freqs).to(dtype), torch.sin(freqs).to(dtype)


def apply_rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, offset=0) -> torch.Tensor:
    """Non-interleaved (rotate-halves) RoPE on ``x [B, L, ..., hd]``.

    ``o0 = x0*cos - x1*sin``, ``o1 = x0*sin + x1*cos`` with the halves split at
    ``rotary_dim/2`` and positions ``offset + arange(L)`` (``offset`` an int or
    a per-batch tensor): based/ops/triton/rotary.py:68-71, :75-105.
    Computed in fp32 and cast back to ``x.dtype`` like that kernel.
    """
    B, L = x.shape[0], x.shape[1]
    half = cos.shape[-1]
    if torch.is_tensor(offset):
        pos = offset.view(B, 1).long() + torch.arange(L).view(1, L)
    else:
        pos = (int(offset) + torch.arange(L)).view(1, L).expand(B, L)
    c = cos[pos].float()
    s = sin[pos].float()
    while c.dim() < x.dim():
        c, s = c.unsqueeze(-2), s.unsqueeze(-2)
    xf = x.float()
    x0, x1, rest = xf[..., :half], xf[..., half : 2 * half], xf[..., 2 * half :]
    out = torch.cat([x0 * c - x1 * s, x0 * s + x1 * c, rest], dim=-1)
    return out.to(x.dtype)


# --------------------------------------------------------------------------
# SlidingAttention: windowed causal softmax attention
# --------------------------------------------------------------------------
def swa_prefill(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    window_left: int,
    softmax_scale: Optional[float] = None,
    q_offset: int = 0,
) -> torch.Tensor:
    """Windowed causal softmax attention.

    q ``[B, Lq, H, hd]``; k, v ``[B, Lk, H, hd]``; query ``i`` sits at key
    position ``i + (Lk - Lq)`` (flash-attn aligns the causal mask to the
    bottom-right corner) and sees keys ``[pos - window_left, pos]`` inclusive.
    Returns ``[B, Lq, H, hd]`` in ``q.dtype``; softmax in fp32 or higher.

    Restates the call sites slide_attention.py:100-106 and :206-213
    (``causal=True``, ``window_size=(window_size//2, 0)`` from :336, window
    semantics comment :97) with the scale from gpt.py:100-104
    (``head_dim**-0.5`` when none is given).
    """
    B, Lq, H, hd = q.shape
    Lk = k.shape[1]
    scale = hd ** -0.5 if softmax_scale is None else softmax_scale
    acc = torch.float64 if q.dtype == torch.float64 else torch.float32
    qf, kf, vf = q.to(acc), k.to(acc), v.to(acc)
    s = torch.einsum("bqhd,bkhd->bhqk", qf, kf) * scale
    qpos = torch.arange(Lq).view(Lq, 1) + (Lk - Lq) + q_offset
    kpos = torch.arange(Lk).view(1, Lk)
    mask = (kpos <= qpos) & (kpos >= qpos - window_left)
    s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("bhqk,bkhd->bqhd", p, vf)
    return o.to(q.dtype)


def swa_decode_step(
    q: torch.Tensor,
    k_new: torch.Tensor,
    v_new: torch.Tensor,
    kv_cache: torch.Tensor,
    cache_seqlens,
    window_left: int,
    softmax_scale: Optional[float] = None,
    cos: Optional[torch.Tensor] = None,
    sin: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """One decode step against the full-length KV cache; appends IN PLACE.

    q ``[B, 1, H, hd]``; k_new, v_new ``[B, 1, H, hd]``; ``kv_cache
    [B, maxL, 2, H, hd]`` (slide_attention.py:374-377); ``cache_seqlens`` an
    int or ``[B]`` tensor: the number of tokens already cached, which is also
    the position of the new token.  With ``cos``/``sin`` given, q and k_new
    are rotated at that position before the append (non-interleaved).

    Restates ``_apply_rotary_update_kvcache_attention``
    (slide_attention.py:384-428) / ``_update_kvcache_attention`` (:465-481):
    append k, v at ``cache_seqlens``, then attend causally over keys
    ``[pos - window_left, pos]``.
    """
    B, _, H, hd = q.shape
    lens = (
        cache_seqlens.long()
        if torch.is_tensor(cache_seqlens)
        else torch.full((B,), int(cache_seqlens), dtype=torch.long)
    )
    if cos is not None:
        q = apply_rotary(q, cos, sin, lens)
        k_new = apply_rotary(k_new, cos, sin, lens)
    out = torch.empty_like(q)
    for b in range(B):
        p = int(lens[b])
        kv_cache[b, p, 0] = k_new[b, 0].to(kv_cache.dtype)
        kv_cache[b, p, 1] = v_new[b, 0].to(kv_cache.dtype)
        lo = max(0, p - window_left)
        kk = kv_cache[b, lo : p + 1, 0].unsqueeze(0)
        vv = kv_cache[b, lo : p + 1, 1].unsqueeze(0)
        out[b : b + 1] = swa_prefill(
            q[b : b + 1], kk.to(q.dtype), vv.to(q.dtype), window_left, softmax_scale
        )
    return out


# --------------------------------------------------------------------------
# BaseConv: gated short causal convolution
#   based/models/mixers/convolution.py:16-217; pinned by tests/golden/baseconv.npz
def gated_conv_prefill(u: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``v = silu(causal_depthwise_conv(u1)) * u2`` with ``u1, u2 = split(u)`` over the last dim.

    u ``[B, L, 2*di]`` (the output of in_proj, convolution.py:205-206), weight ``[di, k]``
    (``conv.weight`` squeezed, :37-44), bias ``[di]`` or None.  The convolution is
    nn.Conv1d with groups = channels and padding k-1 truncated to L (:84), i.e.
    ``c[b, l, ch] = sum_j weight[ch, j] * u1[b, l - (k-1) + j, ch]`` with zeros before the
    start; then silu (:208-210) and the gate (:211).
    """
    B, L, two_di = u.shape
    di, k = weight.shape
    assert two_di == 2 * di
    u1, u2 = u[..., :di], u[..., di:]
    c = torch.zeros(B, L, di, dtype=u.dtype)
    for j in range(k):
        shift = k - 1 - j  # tap j looks `shift` tokens back
        if shift < L:
            c[:, shift:, :] += weight[:, j].to(u.dtype) * u1[:, : L - shift, :]
    if bias is not None:
        c = c + bias.to(u.dtype)
    return torch.nn.functional.silu(c) * u2


def conv_state_from_prompt(u1: torch.Tensor, k: int) -> torch.Tensor:
    """State ``[B, di, k]`` after a prompt: the last k inputs of the convolution, oldest first,
    zeros in front when the prompt is shorter than k (convolution.py:63-67, allocation :111-119)."""
    B, L, di = u1.shape
    state = torch.zeros(B, di, k, dtype=u1.dtype)
    n = min(k, L)
    state[..., k - n:] = u1[:, L - n:, :].transpose(1, 2)
    return state


def gated_conv_step(u_t: torch.Tensor, state: torch.Tensor, weight: torch.Tensor,
                    bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One decode step; ``state [B, di, k]`` is updated IN PLACE.

    u_t ``[B, 2*di]``.  The state is shifted left by one, the new input goes last, the
    output is the dot product with the taps (convolution.py:104-107), then silu and the
    gate (:208-211).  The reference's step ignores the convolution bias on this path
    (:106); with the default ``conv_bias=False`` there is none.  ``bias`` is applied
    here when given so that step and prefill agree.
    """
    di, k = weight.shape
    u1, u2 = u_t[..., :di], u_t[..., di:]
    state.copy_(torch.roll(state, shifts=-1, dims=-1))
    state[:, :, -1] = u1
    c = (state * weight.to(state.dtype)).sum(-1)
    if bias is not None:
        c = c + bias.to(c.dtype)
    return torch.nn.functional.silu(c).to(u_t.dtype) * u2


def baseconv_forward(params: dict, x: torch.Tensor, state: Optional[torch.Tensor] = None,
                     step: bool = False) -> torch.Tensor:
    """BaseConv.forward (convolution.py:197-213): in_proj, gated convolution, out_proj.
    ``params``: in_w, in_b, conv_w ``[di, 1, k]``, out_w, out_b.  With ``state`` given and
    ``step`` false the state is filled from the prompt; with ``step`` true x is ``[B, 1, d]``."""
    w = params["conv_w"].reshape(params["conv_w"].shape[0], -1)
    u = x @ params["in_w"].T + params["in_b"]
    if step:
        v = gated_conv_step(u[:, 0], state, w).unsqueeze(1)
    else:
        v = gated_conv_prefill(u, w)
        if state is not None:
            state.copy_(conv_state_from_prompt(u[..., : w.shape[0]], w.shape[1]))
    return v @ params["out_w"].T + params["out_b"]


# --------------------------------------------------------------------------
# Residual add + RMSNorm, gated MLP activation; pinned by tests/golden/norm_mlp.npz
def add_rmsnorm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                residual: Optional[torch.Tensor] = None, eps: float = 1e-6,
                residual_dtype: Optional[torch.dtype] = None,
                round_input: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """``z = x + residual``; ``out = z / sqrt(mean(z^2) + eps) * weight (+ bias)``; returns
    ``(out, z)`` (the prenorm pair).  Restates rms_norm_ref with ``prenorm=True``
    (based/ops/triton/layer_norm.py:74-125: the sum :110-113, rstd :114, scaling :115) as
    Block.forward uses it (based/models/block.py:134-163).  ``z`` is returned in
    ``residual_dtype`` (default: x's dtype) and the norm sees it as stored, which is what
    ``residual_in_fp32`` selects in the reference.  ``round_input`` rounds z to x's dtype before
    the norm: the unfused ``norm(residual.to(weight.dtype))`` of block.py:134-137.
    """
    rd = residual_dtype or x.dtype
    z = x.to(torch.float64) if x.dtype == torch.float64 else x.float()
    if residual is not None:
        z = z + residual.to(z.dtype)
    z_st = z.to(rd)
    zz = z_st.to(z.dtype)
    if round_input:
        zz = zz.to(x.dtype).to(z.dtype)
    rstd = 1.0 / torch.sqrt(zz.square().mean(dim=-1, keepdim=True) + eps)
    out = zz * rstd * weight.to(z.dtype)
    if bias is not None:
        out = out + bias.to(z.dtype)
    return out.to(x.dtype), z_st


def gated_act(y: torch.Tensor, activation: str = "silu") -> torch.Tensor:
    """``first_half * act(second_half)`` over the last dim: GatedMlp.forward between fc1 and fc2
    (based/models/mlp.py:141-154; "silu" is the SwiGLU case :148-153, "sigmoid" is F.glu :146-147)."""
    a, g = y.chunk(2, dim=-1)
    if activation == "silu":
        return a * torch.nn.functional.silu(g)
    if activation == "sigmoid":
        return a * torch.sigmoid(g)
    raise ValueError(activation)


# --------------------------------------------------------------------------
# Whole model (conv / linear-attention blocks); pinned by tests/golden/full_model.npz
def model_forward(sd: dict, input_ids: torch.Tensor, n_layer: int, n_head: int, linattn_layers,
                  feature_dim: int = 16, eps: float = 1e-5) -> torch.Tensor:
    """Logits of the prenorm block stack on a whole sequence, from a reference state dict.

    Restates GPTModel.forward / GPTLMHeadModel.forward (based/models/gpt.py:639-733, :794-830)
    with Block.forward's prenorm path (based/models/block.py:134-163): embedding; per block
    ``residual += hidden`` -> RMSNorm -> mixer -> ``residual += hidden`` -> RMSNorm -> SwiGLU MLP;
    final add + RMSNorm; tied lm_head.  Layers listed in ``linattn_layers`` are LinearAttention,
    the others BaseConv (the sliding-window mixer has its own oracle functions above).
    """
    h = sd["transformer.embeddings.word_embeddings.weight"][input_ids]
    residual = None
    d = h.shape[-1]
    for i in range(n_layer):
        p = f"transformer.layers.{i}."
        x, residual = add_rmsnorm(h, sd[p + "norm1.weight"], residual=residual, eps=eps)
        if i in linattn_layers:
            x, _, _ = linattn_mixer_forward(x, sd[p + "mixer.proj_q.weight"], sd[p + "mixer.proj_k.weight"],
                                            sd[p + "mixer.proj_v.weight"], sd[p + "mixer.out_proj.weight"],
                                            n_head, feature_dim, d // n_head)
        else:
            x = baseconv_forward({"in_w": sd[p + "mixer.in_proj.weight"], "in_b": sd[p + "mixer.in_proj.bias"],
                                  "conv_w": sd[p + "mixer.conv.conv.weight"], "out_w": sd[p + "mixer.out_proj.weight"],
                                  "out_b": sd[p + "mixer.out_proj.bias"]}, x)
        x, residual = add_rmsnorm(x, sd[p + "norm2.weight"], residual=residual, eps=eps)
        h = gated_act(x @ sd[p + "mlp.fc1.weight"].T, "silu") @ sd[p + "mlp.fc2.weight"].T
    h, _ = add_rmsnorm(h, sd["transformer.ln_f.weight"], residual=residual, eps=eps)
    return h @ sd["transformer.embeddings.word_embeddings.weight"].T
