"""Drop-in ``BaseConv`` / ``ShortConvolution`` mixers on the B200 kernels.

Same constructors, ``forward`` / ``step`` / ``allocate_inference_cache`` signatures, parameter
names and shapes (``in_proj``, ``out_proj``, ``conv.conv`` an ``nn.Conv1d`` with groups =
channels) and state layout (``{"conv": [B, d_inner, k]}`` under ``layer_idx``, nested keys for
``(layer_idx, "conv")``) as based/models/mixers/convolution.py:16-217 of the reference, so
reference checkpoints load.  ``in_proj`` / ``out_proj`` stay ``nn.Linear`` (cuBLAS); the
convolution, the silu and the gate between them are one call into the CUDA library, which
reads the two halves of ``in_proj``'s output in place.  CUDA tensors only.
"""
import torch
import torch.nn as nn

from .. import ops


class ShortConvolution(nn.Module):
    """Depthwise causal convolution over the sequence, dimension last (convolution.py:16-172).

    On its own ``forward`` returns the plain convolution (no activation), like the reference's
    torch path; :class:`BaseConv` calls the fused gated form instead.
    """

    def __init__(self, d_model: int, kernel_size: int, layer_idx=None, use_cuda: bool = False,
                 conv_bias: bool = False, **kwargs):
        super().__init__()
        self.d_model = d_model
        self.kernel_size = kernel_size
        self.layer_idx = layer_idx
        self.use_cuda = use_cuda  # accepted for signature parity; the CUDA library is always used
        self.conv = nn.Conv1d(in_channels=d_model, out_channels=d_model, kernel_size=kernel_size, groups=d_model,
                              padding=kernel_size - 1, bias=conv_bias)

    # ---- state bookkeeping (convolution.py:111-172)
    def allocate_inference_cache(self, batch_size: int, max_seqlen: int, dtype=None, **kwargs):
        return torch.zeros(batch_size, self.d_model, self.kernel_size, device=self.conv.weight.device,
                           dtype=self.conv.weight.dtype if dtype is None else dtype)

    def _init_state(self, inference_params, layer_idx=None, key_value_memory_dict=None):
        if key_value_memory_dict is None:
            key_value_memory_dict = inference_params.key_value_memory_dict
        if layer_idx is None:
            layer_idx = self.layer_idx
        if isinstance(layer_idx, (int, str)):
            if layer_idx not in key_value_memory_dict:
                key_value_memory_dict[layer_idx] = self.allocate_inference_cache(
                    batch_size=inference_params.max_batch_size, max_seqlen=inference_params.max_seqlen)
            else:  # keep the tensor (a captured CUDA graph may hold its address), clear its content
                key_value_memory_dict[layer_idx].zero_()
        else:
            if layer_idx[0] not in key_value_memory_dict:
                key_value_memory_dict[layer_idx[0]] = {}
            self._init_state(inference_params, layer_idx[1], key_value_memory_dict[layer_idx[0]])

    def _get_state(self, inference_params, layer_idx=None):
        if layer_idx is None:
            layer_idx = self.layer_idx
        if isinstance(layer_idx, (int, str)):
            return inference_params.key_value_memory_dict[layer_idx]
        return self._get_state(inference_params, layer_idx[0])[layer_idx[1]]

    def _prefill_state(self, inference_params, batch):
        """The state tensor to fill during a prompt pass, or None outside inference."""
        if inference_params is None:
            return None
        self._init_state(inference_params)
        state = self._get_state(inference_params)
        return state[:batch] if state.shape[0] != batch else state

    # ---- gated form used by BaseConv: u = [u1 | u2] -> silu(conv(u1)) * u2
    def gated(self, u: torch.Tensor, inference_params=None) -> torch.Tensor:
        if inference_params is not None and inference_params.seqlen_offset > 0:
            state = self._get_state(inference_params)
            return ops.gated_conv_step(u, state, self.conv.weight, self.conv.bias).unsqueeze(1)
        state = self._prefill_state(inference_params, u.shape[0])
        if state is not None and (state.dtype != u.dtype or not state.is_contiguous()):
            tmp = torch.empty(state.shape, dtype=u.dtype, device=u.device)
            v = ops.gated_conv_prefill(u, self.conv.weight, self.conv.bias, state=tmp)
            state.copy_(tmp)
            return v
        return ops.gated_conv_prefill(u, self.conv.weight, self.conv.bias, state=state)

    # ---- plain convolution, for callers that use the module directly (convolution.py:47-109)
    def forward(self, x: torch.Tensor, inference_params=None, **kwargs):
        b, l, d = x.shape
        if inference_params is not None:
            if inference_params.seqlen_offset > 0:
                return self.step(x, self._get_state(inference_params))
            state = self._prefill_state(inference_params, b)
            k = min(self.kernel_size, l)
            state.zero_()
            state[..., -k:] = x[:, -k:].transpose(1, 2)
        return self.conv(x.transpose(1, 2))[..., :l].transpose(1, 2)

    def step(self, x: torch.Tensor, state: torch.Tensor):
        state.copy_(torch.roll(state, shifts=-1, dims=-1))
        state[:, :, -1] = x.squeeze(1)
        return torch.einsum("bdk,dgk->bd", state, self.conv.weight).to(x.dtype).unsqueeze(1)


class BaseConv(nn.Module):
    """in_proj -> gated short convolution -> out_proj (convolution.py:174-217)."""

    def __init__(self, d_model: int, l_max: int, kernel_size: int = 3, layer_idx: int = None, use_bias=True,
                 expand_proj: int = 2, use_cuda: bool = False, device=None, dtype=None, **kwargs):
        super().__init__()
        self.d_model = d_model
        self.l_max = l_max
        self.layer_idx = layer_idx
        self.d_inner = expand_proj * self.d_model // 2
        fk = {"device": device, "dtype": dtype}
        self.in_proj = nn.Linear(self.d_model, expand_proj * self.d_model, bias=use_bias, **fk)
        self.out_proj = nn.Linear(self.d_inner, self.d_model, bias=use_bias, **fk)
        self.use_cuda = use_cuda
        self.conv = ShortConvolution(self.d_inner, kernel_size=kernel_size, use_cuda=use_cuda,
                                     layer_idx=(layer_idx, "conv"))
        if device is not None or dtype is not None:
            self.conv.to(device=device, dtype=dtype)

    def forward(self, u, position_ids=None, inference_params=None, *args, **kwargs):
        """u ``[B, L, d_model]`` -> ``[B, L, d_model]``; with ``inference_params`` the prompt pass
        fills the convolution state and later single-token calls step it."""
        if inference_params is not None and inference_params.seqlen_offset > 0:
            state = self.conv._get_state(inference_params)
            if (ops.DECODE_LINEAR_USE["conv"] and ops._decode_rows(u, self.in_proj.weight)
                    and state.dtype == torch.bfloat16 and state.is_contiguous()
                    and state.shape[0] == u.shape[0] and u.shape[1] == 1 and self.d_inner % 8 == 0):
                # decode step: in_proj, the convolution step on the state, silu and the gate in one launch
                v = ops.decode_linear(u, self.in_proj.weight, self.in_proj.bias, epilogue="conv", conv_state=state,
                                      conv_weight=self.conv.conv.weight, conv_bias=self.conv.conv.bias)
                return ops.linear(v, self.out_proj.weight, self.out_proj.bias)
        u = ops.linear(u, self.in_proj.weight, self.in_proj.bias)
        v = self.conv.gated(u, inference_params=inference_params)
        return ops.linear(v, self.out_proj.weight, self.out_proj.bias)

    def allocate_inference_cache(self, batch_size: int, max_seqlen: int, dtype=None, **kwargs):
        return {"conv": self.conv.allocate_inference_cache(batch_size, max_seqlen, dtype=dtype, **kwargs)}
