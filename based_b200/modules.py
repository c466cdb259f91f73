"""Drop-in ``RMSNorm`` and ``GatedMlp`` on the B200 kernels.

Same constructors, parameter names / shapes and ``forward`` signatures as
based/ops/triton/layer_norm.py:926-953 (``RMSNorm``, whose forward is the fused residual-add +
norm the blocks call with ``prenorm=True``) and based/models/mlp.py:99-157 (``GatedMlp``) of the
reference, so reference checkpoints load.  The GEMMs stay ``nn.Linear`` (cuBLAS); the norm and
the gated activation are calls into the CUDA library.  Inference only (no dropout, no
autograd); CUDA tensors only.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops


class RMSNorm(nn.Module):
    def __init__(self, hidden_size, eps=1e-5, dropout_p=0.0, device=None, dtype=None):
        super().__init__()
        self.eps = eps
        if dropout_p > 0.0:
            raise NotImplementedError("inference-only module: dropout is not supported")
        self.drop = None
        self.weight = nn.Parameter(torch.ones(hidden_size, device=device, dtype=dtype))
        self.register_parameter("bias", None)

    def forward(self, x, residual=None, prenorm=False, residual_in_fp32=False, round_input=False):
        """``round_input`` (not in the reference's signature) rounds ``x + residual`` to x's dtype before the
        norm, which is what a block computes when it adds first and then calls the norm on the cast sum."""
        return ops.add_rmsnorm(x, self.weight, self.bias, residual=residual, eps=self.eps, prenorm=prenorm,
                               residual_in_fp32=residual_in_fp32, round_input=round_input)


class GatedMlp(nn.Module):
    """fc1 -> first_half * act(second_half) -> fc2 (mlp.py:141-157); ``mlp_type='base'`` only."""

    def __init__(self, in_features, hidden_features=None, out_features=None, activation=F.sigmoid, bias1=True,
                 bias2=True, multiple_of=256, return_residual=False, device=None, dtype=None, mlp_type="base",
                 ff_mult=2):
        super().__init__()
        if mlp_type != "base":
            raise NotImplementedError("only the 'base' GatedMlp layout (fc1 -> gate -> fc2) is provided")
        fk = {"device": device, "dtype": dtype}
        out_features = out_features if out_features is not None else in_features
        hidden_features = hidden_features if hidden_features is not None else int(8 * in_features / 3)
        hidden_features = (hidden_features + multiple_of - 1) // multiple_of * multiple_of
        self.return_residual = return_residual
        self.fc1 = nn.Linear(in_features, 2 * hidden_features, bias=bias1, **fk)
        self.activation = activation
        self.fc2 = nn.Linear(hidden_features, out_features, bias=bias2, **fk)

    def forward(self, x):
        if self.activation in (F.sigmoid, torch.sigmoid):
            act = "sigmoid"
        elif self.activation is F.silu:
            act = "silu"
        else:
            raise NotImplementedError("GatedMlp: activation must be F.silu (SwiGLU) or F.sigmoid (GLU)")
        if ops.DECODE_LINEAR_USE["gated"] and ops._decode_rows(x, self.fc1.weight) and self.fc1.weight.shape[0] % 16 == 0:
            # decode step: fc1 and the gated activation in one launch, fc2 in another
            y = ops.decode_linear(x, self.fc1.weight, self.fc1.bias, epilogue="gated", activation=act)
        else:
            y = ops.gated_act(self.fc1(x), act)
        y = ops.linear(y, self.fc2.weight, self.fc2.bias)
        return y if not self.return_residual else (y, x)
