"""Drop-in ``LinearAttention`` mixer on the B200 kernels.

Same constructor, ``forward`` / ``allocate_inference_cache`` signatures, parameter names and
shapes (``proj_q``, ``proj_k``, ``proj_v``, ``out_proj``, all bias-free) and state-cache layout
as based/models/mixers/linear_attention.py:77-272 of the reference, so reference checkpoints
load and ``GPTLMHeadModel.generate`` can drive it.  The projections stay ``nn.Linear``
(cuBLAS); everything between them — feature map, causal linear attention, normaliser, state
hand-off, recurrent step — is one call into the CUDA library.  CUDA tensors only.
"""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..sharding import all_reduce_sum_, head_slice, row_parallel_decode_linear


class FeatureMap(nn.Module):
    """Parent feature map; identity (linear_attention.py:38-50)."""

    def __init__(self, input_dim: int, **kwargs):
        super().__init__()
        self.input_dim = input_dim

    def forward(self, x: torch.Tensor):
        return x


class TaylorExp(FeatureMap):
    """2nd-order Taylor approximation of exp(q.k/sqrt(d)) as a feature map
    (linear_attention.py:52-75).  The mixer below never materialises it: the kernels apply
    it on the fly.  ``forward`` is kept for code that calls the map directly."""

    def __init__(self, input_dim: int, **kwargs):
        super().__init__(input_dim, **kwargs)
        self.r2 = math.sqrt(2)
        self.rd = math.sqrt(input_dim)
        self.rrd = math.sqrt(self.rd)

    def forward(self, x: torch.Tensor):
        x2 = (x.unsqueeze(-1) * x.unsqueeze(-2)).flatten(start_dim=-2) / self.r2
        return torch.cat([x[..., :1] ** 0, x / self.rrd, x2 / self.rd], dim=-1)


class LinearAttention(nn.Module):
    # parallel_implementation values of the reference that denote the same mathematics
    # (linear_attention.py:169-215); all of them run the same CUDA kernel here.
    _SAME_MATH = ("quadratic", "linear", "fla_parallel", "fla_chunk", "b200")

    def __init__(
        self,
        d_model: int,
        feature_map: FeatureMap = TaylorExp,
        l_max: int = 2048,
        feature_dim: int = 16,
        head_dim: int = None,
        num_heads: int = 16,
        eps: float = 1e-12,
        layer_idx: int = None,
        parallel_implementation: str = "quadratic",
        state_dtype: torch.dtype = None,
        process_group=None,
        fuse_qkv: bool = False,
        fused_allreduce: bool = False,
        device=None,
        dtype=None,
        **kwargs,
    ):
        super().__init__()
        if parallel_implementation not in self._SAME_MATH:
            raise ValueError(
                f"Parallel implementation {parallel_implementation} not supported "
                f"(supported: {', '.join(self._SAME_MATH)})")
        if feature_dim != 16:
            raise ValueError("the B200 kernels implement the Taylor map for feature_dim = 16")
        if isinstance(feature_map, type):
            feature_map = feature_map(input_dim=feature_dim)
        if not isinstance(feature_map, TaylorExp) and type(feature_map).__name__ != "TaylorExp":
            raise ValueError("the B200 kernels implement the TaylorExp feature map only")
        self.layer_idx = layer_idx
        self.d_model = d_model
        self.l_max = l_max
        self.eps = eps
        self.parallel_implementation = parallel_implementation
        self.head_dim = self.d_model // num_heads if head_dim is None else head_dim
        # extension (the reference mixer has no tensor parallelism): with a process group this rank owns
        # num_heads / world heads — its slices of proj_q/k/v (column-parallel) and of out_proj (row-parallel)
        # and of the recurrent state — and forward() ends with one all-reduce of the output
        self.process_group = process_group
        self.num_heads_total = num_heads
        if process_group is not None:
            import torch.distributed as dist
            h0, h1 = head_slice(num_heads, dist.get_rank(process_group), dist.get_world_size(process_group))
            num_heads = h1 - h0
        self.num_heads = num_heads
        self.feature_dim = feature_dim
        self.feature_map = feature_map
        # extension: dtype of freshly created prefill states; None = the activations' dtype,
        # which is what the reference's einsum produces (linear_attention.py:221-222)
        self.state_dtype = state_dtype
        # extension: in eval mode run proj_q, proj_k, proj_v as ONE GEMM over their concatenated weights
        # (the parameters stay separate, so reference checkpoints still load)
        self.fuse_qkv = fuse_qkv
        # extension (tensor parallelism only): decode steps run out_proj and the all-reduce as ONE kernel per rank
        # that exchanges partial tiles through peer memory; prompt passes keep GEMM + NCCL
        self.fused_allreduce = fused_allreduce
        fk = {"device": device, "dtype": dtype}
        self.proj_q = nn.Linear(self.d_model, self.feature_dim * self.num_heads, bias=False, **fk)
        self.proj_k = nn.Linear(self.d_model, self.feature_dim * self.num_heads, bias=False, **fk)
        self.proj_v = nn.Linear(self.d_model, self.num_heads * self.head_dim, bias=False, **fk)
        self.out_proj = nn.Linear(self.num_heads * self.head_dim, self.d_model, bias=False, **fk)

    def forward(self, hidden_states: torch.Tensor, inference_params=None, *args, **kwargs):
        """hidden_states ``[B, L, d_model]`` -> ``[B, L, d_model]`` (linear_attention.py:115-150).
        Extra keyword arguments the model passes to every mixer (``position_ids``, ``decay``,
        ``stream``, ``seqlen``) are accepted and ignored, as in the reference."""
        b, l, _ = hidden_states.size()
        if self.fuse_qkv and not self.training:
            # one GEMM for the three projections; q, k, v are column slices of its output (the kernels take
            # strided views), so nothing is copied
            nq = self.feature_dim * self.num_heads
            qkv = ops.linear(hidden_states, self._fused_qkv_weight())
            q, k, v = qkv[..., :nq], qkv[..., nq:2 * nq], qkv[..., 2 * nq:]
        else:
            q, k, v = self.proj_q(hidden_states), self.proj_k(hidden_states), self.proj_v(hidden_states)
        q = q.view(b, l, self.num_heads, self.feature_dim).transpose(1, 2)
        k = k.view(b, l, self.num_heads, self.feature_dim).transpose(1, 2)
        v = v.view(b, l, self.num_heads, self.head_dim).transpose(1, 2)

        self.is_inference = inference_params is not None
        if inference_params is None:
            return self.parallel_forward(hidden_states, q, k, v)
        if inference_params.seqlen_offset > 0:
            kv_state, k_state = self._get_inference_cache(inference_params)
            return self.recurrent_forward(hidden_states, kv_state, k_state, q, k, v)
        cached = inference_params.key_value_memory_dict.get(self.layer_idx)
        if cached is not None and cached[0].shape[0] == b:
            # pre-allocated (CUDA-graph) cache: the kernel writes the states in place
            y, _, _ = self.parallel_forward(hidden_states, q, k, v, kv_state=cached[0], k_state=cached[1])
            return y
        y, kv_state, k_state = self.parallel_forward(hidden_states, q, k, v)
        if cached is not None:
            cached[0].copy_(kv_state)
            cached[1].copy_(k_state)
        else:
            inference_params.key_value_memory_dict[self.layer_idx] = (kv_state, k_state)
        return y

    def _fused_qkv_weight(self):
        """``cat(proj_q.weight, proj_k.weight, proj_v.weight)``, rebuilt when a projection changes
        (in-place update, new storage, dtype or device)."""
        ws = (self.proj_q.weight, self.proj_k.weight, self.proj_v.weight)
        key = tuple((w._version, w.data_ptr(), w.dtype, w.device) for w in ws)
        if getattr(self, "_wqkv_key", None) != key:
            self._wqkv = torch.cat([w.detach() for w in ws], dim=0).contiguous()
            self._wqkv_key = key
        return self._wqkv

    def parallel_forward(self, x, q, k, v, kv_state=None, k_state=None):
        """Whole-sequence path (linear_attention.py:152-227): q, k ``[B, H, L, 16]`` raw,
        v ``[B, H, L, dv]``.  Returns ``out_proj(y)`` and, in inference, the states
        ``[B, H, 1, dv, 273]`` / ``[B, H, 1, 1, 273]``."""
        want_state = getattr(self, "is_inference", False)
        y, kv_state, k_state = ops.linattn_prefill(
            q, k, v, eps=self.eps, return_state=want_state, state_dtype=self.state_dtype,
            kv_state=kv_state, k_state=k_state)
        b, h, l, dv = y.shape
        y = y.permute(0, 2, 1, 3).reshape(b, l, h * dv)  # 'b h l d -> b l (h d)': a view
        out = all_reduce_sum_(self.out_proj(y.to(x.dtype)), self.process_group)
        if want_state:
            return out, kv_state, k_state
        return out

    def recurrent_forward(self, hidden_states, kv_state, k_state, q, k, v, decay=None):
        """One token (linear_attention.py:230-252).  ``q``/``k`` are the RAW ``[B, H, 1, 16]``
        projections: the kernel applies the feature map itself (the reference maps them
        first, :139).  ``kv_state``/``k_state`` are updated in place."""
        b, h, l, d = q.shape
        assert l == 1, f"q.shape is {q.shape} but should be ({b}, {h}, 1, {d})"
        eps = 1e-6 if "fla" in self.parallel_implementation else 1e-12
        y = ops.linattn_decode(q, k, v, kv_state, k_state, eps=eps)
        return row_parallel_decode_linear(self, y, self.out_proj.weight, self.out_proj.bias, self.process_group)

    def expanded_size(self):
        return self.feature_dim ** 2 + self.feature_dim + 1

    def allocate_inference_cache(self, batch_size: int, max_seqlen: int, dtype=None, **kwargs):
        """Zeroed ``(kv_state [B, H, 1, dv, 273], k_state [B, H, 1, 1, 273])``
        (linear_attention.py:258-269)."""
        dev = self.out_proj.weight.device
        kv_shape = (batch_size, self.num_heads, 1, self.head_dim, self.expanded_size())
        k_shape = (batch_size, self.num_heads, 1, 1, self.expanded_size())
        return (torch.zeros(*kv_shape, dtype=dtype, device=dev), torch.zeros(*k_shape, dtype=dtype, device=dev))

    def _get_inference_cache(self, inference_params):
        return inference_params.key_value_memory_dict[self.layer_idx]
