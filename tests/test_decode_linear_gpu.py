"""Decode-step linear layers with fused epilogues (bf16) against fp64 restatements: plain, gated (fc1 + SwiGLU /
GLU) and the BaseConv step (in_proj + conv state update + silu + gate).  Tolerance 2e-2 relative (bf16 I/O)."""
import pytest
import torch

from conftest import rel_err
from oracle import based_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from based_b200 import ops as _ops
    return _ops


def _mk(M, N, K, seed, bias):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) / K ** 0.5).bfloat16()
    b = (torch.randn(N, generator=g) * 0.1).bfloat16() if bias else None
    return x, w, b


@pytest.mark.parametrize("M,N,K,bias", [(16, 1024, 1024, False), (1, 8, 32, True), (5, 264, 96, True), (16, 4096, 1024, False),
                                        (3, 1024, 2048, False), (37, 64, 160, True), (16, 50280, 1024, False)])
def test_decode_linear_plain(ops, M, N, K, bias):
    x, w, b = _mk(M, N, K, M + N + K, bias)
    ref = x.double() @ w.double().T + (0 if b is None else b.double())
    y = ops.decode_linear(x.cuda(), w.cuda(), None if b is None else b.cuda())
    assert y.shape == (M, N) and y.dtype == torch.bfloat16
    assert rel_err(y.cpu().double(), ref) < 2e-2
    # strided rows (a [B, 1, K] slice of a longer buffer) and a leading batch shape
    big = torch.zeros(M, 3, K, dtype=torch.bfloat16, device="cuda")
    big[:, 1] = x.cuda()
    y2 = ops.decode_linear(big[:, 1:2], w.cuda(), None if b is None else b.cuda())
    assert y2.shape == (M, 1, N) and torch.equal(y2[:, 0], y)


@pytest.mark.parametrize("act", ["silu", "sigmoid"])
@pytest.mark.parametrize("M,F,K,bias", [(16, 2048, 1024, False), (2, 8, 64, True), (9, 264, 128, False)])
def test_decode_linear_gated(ops, act, M, F, K, bias):
    x, w, b = _mk(M, 2 * F, K, F + K, bias)
    u = x.double() @ w.double().T + (0 if b is None else b.double())
    ref = O.gated_act(u.bfloat16().double(), act)      # fc1's output is a bf16 tensor before the activation
    y = ops.decode_linear(x.cuda(), w.cuda(), None if b is None else b.cuda(), epilogue="gated", activation=act)
    assert y.shape == (M, F)
    assert rel_err(y.cpu().double(), ref) < 2e-2


@pytest.mark.parametrize("M,di,K,ck,cbias", [(16, 2048, 1024, 3, False), (3, 64, 96, 4, True), (1, 8, 32, 2, False)])
def test_decode_linear_conv_steps(ops, M, di, K, ck, cbias):
    """Three consecutive steps: outputs and the state trajectory equal the oracle's gated_conv_step on in_proj(x)."""
    g = torch.Generator().manual_seed(di + K)
    w = (torch.randn(2 * di, K, generator=g) / K ** 0.5).bfloat16()
    b = (torch.randn(2 * di, generator=g) * 0.1).bfloat16()
    cw = (torch.randn(di, ck, generator=g) * 0.5).bfloat16()
    cb = (torch.randn(di, generator=g) * 0.1).bfloat16() if cbias else None
    state = torch.randn(M, di, ck, generator=g).bfloat16()
    st_dev, st_ref = state.cuda(), state.double()
    for step in range(3):
        x = torch.randn(M, K, generator=g).bfloat16()
        u = (x.double() @ w.double().T + b.double()).bfloat16().double()     # in_proj output as the bf16 tensor it is
        ref = O.gated_conv_step(u, st_ref, cw.double(), None if cb is None else cb.double())
        y = ops.decode_linear(x.cuda(), w.cuda(), b.cuda(), epilogue="conv", conv_state=st_dev, conv_weight=cw.cuda(),
                              conv_bias=None if cb is None else cb.cuda())
        assert y.shape == (M, di)
        assert rel_err(y.cpu().double(), ref) < 2e-2, step
        # the appended input is a rounded GEMM result: compare with tolerance, the shifted part exactly
        assert rel_err(st_dev[..., -1].cpu().double(), st_ref[..., -1]) < 2e-2
        assert torch.equal(st_dev[..., :-1].cpu().double(), st_ref[..., :-1]) or step > 0
        st_ref.copy_(st_dev.cpu().double())   # keep the trajectories aligned for the next step


def test_decode_linear_rejects_what_it_cannot_run(ops):
    from based_b200 import _capi
    x = torch.randn(4, 40, device="cuda").bfloat16()          # K not a multiple of 32
    with pytest.raises(_capi.BasedLibraryError):
        ops.decode_linear(x, torch.randn(16, 40, device="cuda").bfloat16())
    with pytest.raises(_capi.BasedLibraryError):               # outputs not a multiple of 8
        ops.decode_linear(torch.randn(4, 64, device="cuda").bfloat16(), torch.randn(12, 64, device="cuda").bfloat16())
    with pytest.raises(TypeError):
        ops.decode_linear(torch.randn(4, 64, device="cuda"), torch.randn(16, 64, device="cuda"))
