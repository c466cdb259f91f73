"""Residual add + RMSNorm and the gated MLP activation: CUDA kernels through the C ABI against the
CPU oracle and the reference's golden vectors.  Tolerances: relative error 1e-5 (fp32 I/O) and
2e-2 (bf16 I/O) against an fp64 oracle on the same inputs."""
import pytest
import torch
import torch.nn.functional as F

from conftest import load_golden, rel_err
from oracle import based_oracle as O

pytestmark = pytest.mark.gpu
TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2}


@pytest.fixture(scope="module")
def ops():
    from based_b200 import ops as _ops
    return _ops


@pytest.mark.parametrize("io,res32", [(torch.float32, True), (torch.bfloat16, True), (torch.bfloat16, False)])
@pytest.mark.parametrize("M,D,bias", [(5, 64, False), (33, 1024, False), (7, 1792, True), (3, 8, True), (2, 8192, False),
                                      (1, 4104, False)])
def test_add_rmsnorm_vs_oracle(ops, io, res32, M, D, bias):
    g = torch.Generator().manual_seed(M * 31 + D)
    x = torch.randn(2, M, D, generator=g).to(io)
    rd = torch.float32 if res32 else io
    res = (torch.randn(2, M, D, generator=g) * 2).to(rd)
    w = (torch.randn(D, generator=g) * 0.3 + 1).to(io)
    b = (torch.randn(D, generator=g) * 0.1).to(io) if bias else None
    out_ref, z_ref = O.add_rmsnorm(x.double(), w.double(), None if b is None else b.double(), residual=res.double(),
                                   eps=1e-5)
    out, z = ops.add_rmsnorm(x.cuda(), w.cuda(), None if b is None else b.cuda(), residual=res.cuda(), eps=1e-5,
                             prenorm=True, residual_in_fp32=res32)
    assert out.dtype == io and z.dtype == rd and out.shape == x.shape
    assert rel_err(z.cpu().double(), z_ref) < (1e-6 if rd == torch.float32 else 5e-3)
    assert rel_err(out.cpu().double(), out_ref) < TOL[io]
    # first block of a model: no residual yet; and the non-prenorm form returns only the normed tensor
    out0 = ops.add_rmsnorm(x.cuda(), w.cuda(), eps=1e-5)
    assert rel_err(out0.cpu().double(), O.add_rmsnorm(x.double(), w.double(), eps=1e-5)[0]) < TOL[io]
    if rd != torch.float32:
        # the norm is taken of the residual stream as stored (bf16)
        o2, z2 = O.add_rmsnorm(x, w, b, residual=res, eps=1e-5)
        assert torch.equal(z.cpu(), z2)


def test_add_rmsnorm_golden_and_rejections(ops):
    g = {k: torch.as_tensor(v) for k, v in load_golden("norm_mlp.npz").items()}
    x, res, w, b = (g[k].float().cuda() for k in ("x", "residual", "weight", "bias"))
    out, z = ops.add_rmsnorm(x, w, residual=res, eps=1e-5, prenorm=True)
    assert rel_err(out.cpu().double(), g["out_res"]) < 1e-5 and rel_err(z.cpu().double(), g["res_out"]) < 1e-6
    assert rel_err(ops.add_rmsnorm(x, w, eps=1e-5).cpu().double(), g["out_nores"]) < 1e-5
    assert rel_err(ops.add_rmsnorm(x, w, b, residual=res, eps=1e-6).cpu().double(), g["out_bias"]) < 1e-5
    from based_b200 import _capi
    with pytest.raises(_capi.BasedLibraryError):      # D not a multiple of 8
        ops.add_rmsnorm(torch.randn(4, 12, device="cuda"), torch.ones(12, device="cuda"))
    with pytest.raises(_capi.BasedLibraryError):      # D beyond the kernel's row capacity
        ops.add_rmsnorm(torch.randn(2, 8200, device="cuda"), torch.ones(8200, device="cuda"))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("act", ["silu", "sigmoid"])
@pytest.mark.parametrize("M,Fh", [(3, 8), (37, 2816), (5, 4864), (1, 264)])
def test_gated_act_vs_oracle(ops, dtype, act, M, Fh):
    g = torch.Generator().manual_seed(M + Fh)
    y = (torch.randn(2, M, 2 * Fh, generator=g) * 2).to(dtype)
    ref = O.gated_act(y.double(), act)
    out = ops.gated_act(y.cuda(), act)
    assert out.shape == (2, M, Fh) and out.dtype == dtype
    assert rel_err(out.cpu().double(), ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_modules_match_reference_golden(dtype):
    """Drop-in RMSNorm and GatedMlp with the reference's weights (tests/golden/norm_mlp.npz)."""
    from based_b200.modules import GatedMlp, RMSNorm
    g = {k: torch.as_tensor(v) for k, v in load_golden("norm_mlp.npz").items()}
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    n = RMSNorm(g["weight"].numel(), eps=1e-5)
    n.load_state_dict({"weight": g["weight"]})
    n = n.to(device="cuda", dtype=dtype)
    x, res = g["x"].to(device="cuda", dtype=dtype), g["residual"].cuda().float()
    with torch.inference_mode():
        out, z = n(x, residual=res, prenorm=True, residual_in_fp32=True)
        assert z.dtype == torch.float32
        ref_out, ref_z = O.add_rmsnorm(x.cpu().double(), g["weight"].to(dtype).double(), residual=res.cpu().double(),
                                       eps=1e-5)
        assert rel_err(out.cpu().double(), ref_out) < TOL[dtype] and rel_err(z.cpu().double(), ref_z) < 1e-6
        if dtype == torch.float32:
            assert rel_err(out.cpu().double(), g["out_res"]) < 1e-5
        for name, act in (("silu", F.silu), ("sigmoid", F.sigmoid)):
            m = GatedMlp(32, activation=act, bias1=False, bias2=False, multiple_of=32)
            m.load_state_dict({"fc1.weight": g[f"mlp_{name}_fc1"], "fc2.weight": g[f"mlp_{name}_fc2"]})
            m = m.to(device="cuda", dtype=dtype)
            y = m(g[f"mlp_{name}_x"].to(device="cuda", dtype=dtype))
            assert rel_err(y.cpu().double(), g[f"mlp_{name}_y"]) < tol


def test_norm_act_full_size_properties(ops):
    """Row and element independence at the 360M model's sizes (M = 16 x 2048 rows, D = 1024, F = 2816):
    the full launch equals launches over slices, sampled rows equal the oracle, and the norm is
    scale-invariant up to eps."""
    M, D, Fh = 16 * 2048, 1024, 2816
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(M, D, device="cuda", generator=g).bfloat16()
    res = torch.randn(M, D, device="cuda", generator=g)
    w = (torch.randn(D, device="cuda", generator=g) * 0.2 + 1).bfloat16()
    out, z = ops.add_rmsnorm(x, w, residual=res, prenorm=True, residual_in_fp32=True)
    for lo in (0, 12345, M - 64):
        o2, z2 = ops.add_rmsnorm(x[lo:lo + 64], w, residual=res[lo:lo + 64], prenorm=True, residual_in_fp32=True)
        assert torch.equal(o2, out[lo:lo + 64]) and torch.equal(z2, z[lo:lo + 64])
        ref, _ = O.add_rmsnorm(x[lo:lo + 64].cpu().double(), w.cpu().double(), residual=res[lo:lo + 64].cpu().double())
        assert rel_err(out[lo:lo + 64].cpu().double(), ref) < TOL[torch.bfloat16]
    assert torch.equal(z, x.float() + res)
    scaled = ops.add_rmsnorm((x.float() * 4).bfloat16(), w, residual=res * 4, residual_in_fp32=True)
    assert rel_err(scaled.float(), out.float()) < 1e-2
    y = torch.randn(M, 2 * Fh, device="cuda", generator=g).bfloat16()
    h = ops.gated_act(y, "silu")
    assert torch.equal(ops.gated_act(y[777:900], "silu"), h[777:900])
    assert rel_err(h[:64].cpu().double(), O.gated_act(y[:64].cpu().double(), "silu")) < TOL[torch.bfloat16]
