"""Drop-in ``SlidingAttention`` mixer on the B200 kernels.

Same constructor and ``forward`` / ``allocate_inference_cache`` signatures, parameter names
(``Wqkv``, ``out_proj``) and KV-cache layout ``[B, max_seqlen, 2, H, head_dim]`` as
based/models/mixers/slide_attention.py:284-600.  The reference reaches flash-attn for the
attention and the rotary embedding; here both are calls into the CUDA library.  Supported:
self-attention with ``num_heads_kv == num_heads``, non-interleaved rotary without xPos scale,
no dropout (inference).  CUDA tensors only.
"""
import torch
import torch.nn as nn

from .. import ops
from ..sharding import all_reduce_sum_, head_slice, row_parallel_decode_linear


class RotaryEmbedding(nn.Module):
    """cos/sin tables as the reference's rotary module builds them (fp32 ``outer(t, inv_freq)``,
    ``inv_freq = base**(-arange(0, dim, 2)/dim)``, cast to the model dtype)."""

    def __init__(self, dim: int, base=10000.0, interleaved=False, scale_base=None, device=None):
        super().__init__()
        if interleaved or scale_base is not None:
            raise NotImplementedError("only non-interleaved rotary without xPos scaling is implemented")
        self.dim, self.base, self.interleaved, self.scale = dim, float(base), False, None
        self._seq_len_cached = 0
        self._cos_cached = None
        self._sin_cached = None

    def _update_cos_sin_cache(self, seqlen, device=None, dtype=None):
        if (seqlen > self._seq_len_cached or self._cos_cached is None or self._cos_cached.device != device
                or self._cos_cached.dtype != dtype):
            self._seq_len_cached = seqlen
            inv_freq = 1.0 / (self.base ** (torch.arange(0, self.dim, 2, device=device, dtype=torch.float32) / self.dim))
            t = torch.arange(seqlen, device=device, dtype=torch.float32)
            freqs = torch.outer(t, inv_freq)
            self._cos_cached = torch.cos(freqs).to(dtype).contiguous()
            self._sin_cached = torch.sin(freqs).to(dtype).contiguous()

    def forward(self, qkv: torch.Tensor, seqlen_offset=0, max_seqlen=None):
        """In-place RoPE on q and k of packed ``qkv [B, L, 3, H, hd]`` (slide_attention.py:553-556)."""
        L = qkv.shape[1]
        need = max_seqlen if max_seqlen is not None else L + (0 if torch.is_tensor(seqlen_offset) else seqlen_offset)
        self._update_cos_sin_cache(max(need, L), device=qkv.device, dtype=qkv.dtype)
        B, _, three, H, hd = qkv.shape
        if qkv.stride(2) == H * hd and qkv.stride(3) == hd:
            # q and k are adjacent in the packed tensor: one launch over 2H heads
            qk = torch.as_strided(qkv, (B, L, 2 * H, hd), (qkv.stride(0), qkv.stride(1), hd, 1), qkv.storage_offset())
            ops.rotary_apply_(qk, self._cos_cached, self._sin_cached, seqlen_offset)
        else:
            ops.rotary_apply_(qkv[:, :, 0], self._cos_cached, self._sin_cached, seqlen_offset)
            ops.rotary_apply_(qkv[:, :, 1], self._cos_cached, self._sin_cached, seqlen_offset)
        return qkv


class SlidingAttention(nn.Module):
    def __init__(
        self,
        embed_dim,
        num_heads,
        num_heads_kv=None,
        cross_attn=False,
        qkv_proj_bias=True,
        out_proj_bias=True,
        dropout=0.0,
        softmax_scale=None,
        causal=True,
        layer_idx=None,
        rotary_emb_dim=0,
        rotary_emb_base=10000.0,
        rotary_emb_scale_base=None,
        rotary_emb_interleaved=False,
        fused_bias_fc=False,
        use_flash_attn=True,
        return_residual=False,
        checkpointing=False,
        window_size=128,
        process_group=None,
        fused_allreduce=False,
        device=None,
        dtype=None,
    ) -> None:
        super().__init__()
        if cross_attn:
            raise NotImplementedError("cross-attention is not part of the Based path")
        if num_heads_kv is not None and num_heads_kv != num_heads:
            raise NotImplementedError("MQA/GQA (num_heads_kv != num_heads) is not implemented")
        if window_size is None:
            raise ValueError("SlidingAttention needs a window_size")
        factory_kwargs = {"device": device, "dtype": dtype}
        self.embed_dim = embed_dim
        self.cross_attn = False
        self.causal = True  # the reference hard-codes causal attention (slide_attention.py:319)
        self.layer_idx = layer_idx
        self.rotary_emb_dim = rotary_emb_dim
        self.return_residual = return_residual
        self.dropout_p = dropout
        # (left, right) window as the reference stores it: the constructor argument is halved
        self.window = (window_size // 2, 0)
        assert self.embed_dim % num_heads == 0, "embed_dim must be divisible by num_heads"
        self.head_dim = self.embed_dim // num_heads
        # extension (the reference class takes no process group): head-sharded tensor parallelism,
        # Wqkv column-parallel, out_proj row-parallel, one all-reduce of the output
        self.process_group = process_group
        # extension (tensor parallelism only): single-token steps run out_proj and the all-reduce as one kernel
        self.fused_allreduce = fused_allreduce
        self.num_heads_total = num_heads
        if process_group is not None:
            import torch.distributed as dist
            h0, h1 = head_slice(num_heads, dist.get_rank(process_group), dist.get_world_size(process_group))
            num_heads = h1 - h0
        self.num_heads = num_heads
        self.num_heads_kv = num_heads
        self.tp_rank0 = process_group is None or h0 == 0
        self.softmax_scale = softmax_scale
        if self.rotary_emb_dim > 0:
            self.rotary_emb = RotaryEmbedding(self.rotary_emb_dim, base=rotary_emb_base,
                                              scale_base=rotary_emb_scale_base,
                                              interleaved=rotary_emb_interleaved, device=device)
        local = self.num_heads * self.head_dim
        self.Wqkv = nn.Linear(embed_dim, 3 * local, bias=qkv_proj_bias, **factory_kwargs)
        # row-parallel: the bias must be added once, so only the rank owning head 0 keeps it
        self.out_proj = nn.Linear(local, embed_dim, bias=out_proj_bias and self.tp_rank0, **factory_kwargs)

    def allocate_inference_cache(self, batch_size, max_seqlen, dtype=None):
        dtype = self.out_proj.weight.dtype if dtype is None else dtype
        return torch.empty(batch_size, max_seqlen, 2, self.num_heads_kv, self.head_dim, dtype=dtype,
                           device=self.out_proj.weight.device)

    def _kv_cache(self, inference_params, like):
        """The layer's cache, created on first use like the reference's _update_kv_cache
        (slide_attention.py:255-281)."""
        assert self.layer_idx is not None, "Generation requires layer_idx in the constructor"
        d = inference_params.key_value_memory_dict
        if self.layer_idx not in d:
            d[self.layer_idx] = torch.empty(inference_params.max_batch_size, inference_params.max_seqlen, 2,
                                            self.num_heads_kv, self.head_dim, dtype=like.dtype, device=like.device)
        return d[self.layer_idx]

    def forward(self, x, x_kv=None, key_padding_mask=None, cu_seqlens=None, max_seqlen=None, mixer_subset=None,
                inference_params=None, **kwargs):
        """x ``[B, L, embed_dim]`` -> ``[B, L, embed_dim]`` (slide_attention.py:483-600)."""
        if x_kv is not None or key_padding_mask is not None or cu_seqlens is not None or mixer_subset is not None:
            raise NotImplementedError("only the dense self-attention path of the Based model is implemented")
        if self.training and self.dropout_p > 0:
            raise NotImplementedError("attention dropout is not implemented (inference kernels)")
        batch, seqlen = x.shape[:2]
        qkv = ops.linear(x, self.Wqkv.weight, self.Wqkv.bias)
        in_dtype = qkv.dtype
        if in_dtype == torch.float16:
            raise TypeError("float16 is not supported by the B200 kernels; use bfloat16")
        if in_dtype != torch.bfloat16:
            qkv = qkv.to(torch.bfloat16)  # the reference's inner attention does the same cast (:76-78)
        qkv = qkv.view(batch, seqlen, 3, self.num_heads, self.head_dim)
        w = self.window[0]

        if inference_params is None or inference_params.seqlen_offset == 0:
            cache = None
            if inference_params is not None:
                cache = self._kv_cache(inference_params, qkv)
                b0 = inference_params.batch_size_offset
                assert b0 + batch <= cache.shape[0] and seqlen <= cache.shape[1]
            if (cache is not None and self.rotary_emb_dim == self.head_dim and cache.dtype == torch.bfloat16
                    and self.head_dim % 16 == 0):
                # rotary on q, k and the cache fill in one pass over the packed projection
                self.rotary_emb._update_cos_sin_cache(max(inference_params.max_seqlen, seqlen), device=qkv.device,
                                                      dtype=qkv.dtype)
                ops.rotary_qkv_cache_(qkv, self.rotary_emb._cos_cached, self.rotary_emb._sin_cached,
                                      cache[b0:b0 + batch])
            else:
                if self.rotary_emb_dim > 0:
                    rmax = inference_params.max_seqlen if inference_params is not None else None
                    qkv = self.rotary_emb(qkv, seqlen_offset=0, max_seqlen=rmax)
                if cache is not None:
                    cache[b0:b0 + batch, :seqlen] = qkv[:, :, 1:].to(cache.dtype)
            context = ops.swa_prefill(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], w, self.softmax_scale)
        else:
            cache = self._kv_cache(inference_params, qkv)[:batch]
            if cache.dtype != torch.bfloat16:
                raise TypeError("decode needs a bfloat16 KV cache")
            lens = inference_params.lengths_per_sample
            lens = lens[:batch] if lens is not None else inference_params.seqlen_offset
            cos = sin = None
            if self.rotary_emb_dim > 0:
                self.rotary_emb._update_cos_sin_cache(inference_params.max_seqlen, device=qkv.device, dtype=qkv.dtype)
                cos, sin = self.rotary_emb._cos_cached, self.rotary_emb._sin_cached
            context = ops.swa_decode(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], cache, lens, w, self.softmax_scale,
                                     rotary_cos=cos, rotary_sin=sin)
        context = context.to(in_dtype).reshape(batch, seqlen, self.num_heads * self.head_dim)
        if seqlen == 1 and inference_params is not None and inference_params.seqlen_offset > 0:
            out = row_parallel_decode_linear(self, context, self.out_proj.weight, self.out_proj.bias, self.process_group)
        else:
            out = all_reduce_sum_(ops.linear(context, self.out_proj.weight, self.out_proj.bias), self.process_group)
        return out if not self.return_residual else (out, x)
