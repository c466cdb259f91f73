"""Gated short convolution (BaseConv): CUDA kernels through the C ABI against the CPU oracle and
the reference's golden vectors.  Tolerances: relative error 1e-5 for fp32 I/O (fp32 arithmetic,
fast exp) and 2e-2 for bf16 I/O, against an fp64 oracle on the same inputs."""
import pytest
import torch

from conftest import load_golden, rel_err
from oracle import based_oracle as O

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2}


@pytest.fixture(scope="module")
def ops():
    from based_b200 import ops as _ops
    return _ops


def _case(B, L, di, k, dtype, bias, seed):
    g = torch.Generator().manual_seed(seed)
    u = torch.randn(B, L, 2 * di, generator=g).to(dtype)
    w = (torch.randn(di, k, generator=g) * 0.5).to(dtype)
    b = (torch.randn(di, generator=g) * 0.1).to(dtype) if bias else None
    return u, w, b


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,L,di,k,bias", [(2, 37, 64, 3, False), (1, 1, 8, 3, False), (3, 2, 16, 3, True),
                                           (2, 33, 1032, 3, False), (1, 130, 256, 4, True), (2, 65, 128, 2, False),
                                           (1, 31, 64, 1, True), (2, 32, 64, 3, False)])
def test_gated_conv_prefill_vs_oracle(ops, dtype, B, L, di, k, bias):
    u, w, b = _case(B, L, di, k, dtype, bias, seed=L * 7 + di + k)
    ref = O.gated_conv_prefill(u.double(), w.double(), None if b is None else b.double())
    st_ref = O.conv_state_from_prompt(u[..., :di].double(), k)
    state = torch.full((B, di, k), 7.0, dtype=dtype, device="cuda")
    v = ops.gated_conv_prefill(u.cuda(), w.cuda(), None if b is None else b.cuda(), state=state)
    assert v.shape == (B, L, di)
    assert rel_err(v.cpu(), ref) < TOL[dtype]
    assert torch.equal(state.cpu().double(), st_ref)          # a copy of the inputs: exact
    v2 = ops.gated_conv_prefill(u.cuda(), w.cuda(), None if b is None else b.cuda())  # no state requested
    assert torch.equal(v2, v)


def test_gated_conv_prefill_strided_views_and_fp32_taps(ops):
    """u as a slice of a wider buffer, output into a strided view, fp32 taps with bf16 activations."""
    B, L, di, k = 2, 50, 64, 3
    g = torch.Generator().manual_seed(5)
    big = torch.randn(B, L + 3, 2 * di + 16, generator=g).bfloat16().cuda()
    u = big[:, 2:L + 2, 8:8 + 2 * di]
    w = (torch.randn(di, 1, k, generator=g) * 0.5).cuda()       # nn.Conv1d layout, fp32
    out = torch.zeros(B, L, 2 * di, dtype=torch.bfloat16, device="cuda")
    v = ops.gated_conv_prefill(u, w, out=out[..., di:])
    ref = O.gated_conv_prefill(u.cpu().double(), w.cpu().double().reshape(di, k))
    assert rel_err(v.cpu(), ref) < TOL[torch.bfloat16]
    assert (out[..., :di] == 0).all()
    from based_b200 import _capi
    with pytest.raises(_capi.BasedLibraryError):                # channel offset not a multiple of 8
        ops.gated_conv_prefill(big[:, :L, 4:4 + 2 * di], w)
    with pytest.raises(_capi.BasedLibraryError):                # kernel size beyond 4
        ops.gated_conv_prefill(u, torch.randn(di, 5, device="cuda"))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("k,bias", [(3, False), (4, True), (2, False)])
def test_gated_conv_steps_continue_the_prefill(ops, dtype, k, bias):
    """prefill(L) then n single-token steps == prefill(L + n) on the last n tokens; states agree."""
    B, L, n, di = 3, 21, 5, 96
    u, w, b = _case(B, L + n, di, k, dtype, bias, seed=k)
    uc, wc, bc = u.cuda(), w.cuda(), None if b is None else b.cuda()
    full_state = torch.empty(B, di, k, dtype=dtype, device="cuda")
    full = ops.gated_conv_prefill(uc, wc, bc, state=full_state)
    state = torch.empty(B, di, k, dtype=dtype, device="cuda")
    ops.gated_conv_prefill(uc[:, :L], wc, bc, state=state)
    st_or = O.conv_state_from_prompt(u[:, :L, :di].double(), k)
    for i in range(n):
        y = ops.gated_conv_step(uc[:, L + i], state, wc, bc)
        y_or = O.gated_conv_step(u[:, L + i].double(), st_or, w.double(), None if b is None else b.double())
        assert rel_err(y.cpu(), y_or) < TOL[dtype]
        assert rel_err(y.float(), full[:, L + i].float()) < (1e-6 if dtype == torch.float32 else 1e-2)
        assert torch.equal(state.cpu().double(), st_or)
    assert torch.equal(state, full_state)
    # a prompt shorter than the kernel leaves leading zeros, and stepping from it still works
    short = torch.full((B, di, k), 3.0, dtype=dtype, device="cuda")
    ops.gated_conv_prefill(uc[:, :1], wc, bc, state=short)
    assert (short[..., : k - 1] == 0).all() and torch.equal(short[..., -1], uc[:, 0, :di])


def test_gated_conv_golden(ops):
    """Vectors the reference's BaseConv produced (fp64 run), kernel in fp32."""
    g = load_golden("baseconv.npz")
    u = torch.as_tensor(g["u"]).float().cuda()
    w = torch.as_tensor(g["conv_w"]).float().cuda()
    state = torch.empty(u.shape[0], w.shape[0], w.shape[2], device="cuda")
    v = ops.gated_conv_prefill(u, w, state=state)
    assert rel_err(v.cpu().double(), torch.as_tensor(g["v"])) < TOL[torch.float32]
    assert rel_err(state.cpu().double(), torch.as_tensor(g["state_prefill"])) < 1e-7


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_baseconv_mixer_matches_reference_golden(dtype):
    """The drop-in BaseConv with the reference's weights: train path, prompt pass + state, three
    decode steps, short prompt (tests/golden/baseconv.npz)."""
    from based_b200.generation import InferenceParams
    from based_b200.mixers import BaseConv
    g = {k: torch.as_tensor(v) for k, v in load_golden("baseconv.npz").items()}
    d = g["x"].shape[-1]
    m = BaseConv(d_model=d, l_max=128, kernel_size=3, layer_idx=0)
    m.load_state_dict({"in_proj.weight": g["in_w"], "in_proj.bias": g["in_b"], "conv.conv.weight": g["conv_w"],
                       "out_proj.weight": g["out_w"], "out_proj.bias": g["out_b"]})
    m = m.to(device="cuda", dtype=dtype)
    tol = 1e-4 if dtype == torch.float32 else 3e-2   # fp32 GEMMs may run in TF32-free fp32; bf16 adds GEMM rounding
    x = g["x"].to(device="cuda", dtype=dtype)
    with torch.inference_mode():
        assert rel_err(m(x).cpu().double(), g["y_train"]) < tol
        ip = InferenceParams(max_seqlen=128, max_batch_size=x.shape[0])
        assert rel_err(m(x, inference_params=ip).cpu().double(), g["y_prefill"]) < tol
        state = ip.key_value_memory_dict[0]["conv"]
        assert state.shape == g["state_prefill"].shape
        assert rel_err(state.cpu().double(), g["state_prefill"]) < tol
        for i in range(3):
            ip.seqlen_offset = x.shape[1] + i
            y = m(g[f"x_step{i}"].to(device="cuda", dtype=dtype), inference_params=ip)
            assert y.shape == g[f"y_step{i}"].shape
            assert rel_err(y.cpu().double(), g[f"y_step{i}"]) < tol
            assert rel_err(state.cpu().double(), g[f"state_step{i}"]) < tol
        ip2 = InferenceParams(max_seqlen=128, max_batch_size=x.shape[0])
        ys = m(g["x_short"].to(device="cuda", dtype=dtype), inference_params=ip2)
        assert rel_err(ys.cpu().double(), g["y_short"]) < tol
        assert rel_err(ip2.key_value_memory_dict[0]["conv"].cpu().double(), g["state_short"]) < tol


def test_gated_conv_full_size_properties(ops):
    """B=16, L=2048, d_inner=1024 bf16 (the 360M model's BaseConv layer at the generation benchmark's
    prompt size): sampled rows against the oracle, state == last inputs, step == longer prefill."""
    B, L, di, k = 16, 2048, 1024, 3
    g = torch.Generator(device="cuda").manual_seed(0)
    u = torch.randn(B, L + 1, 2 * di, device="cuda", generator=g).bfloat16()
    w = (torch.randn(di, k, device="cuda", generator=g) * 0.5).bfloat16()
    state = torch.empty(B, di, k, dtype=torch.bfloat16, device="cuda")
    v = ops.gated_conv_prefill(u[:, :L], w, state=state)
    assert torch.equal(state, u[:, L - k:L, :di].transpose(1, 2))
    for b, l0 in ((0, 0), (7, 1000), (15, L - 40)):
        ref = O.gated_conv_prefill(u[b:b + 1, max(l0 - 2, 0):l0 + 40].cpu().double(), w.cpu().double())
        off = l0 - max(l0 - 2, 0)
        assert rel_err(v[b:b + 1, l0:l0 + 40].cpu(), ref[:, off:]) < TOL[torch.bfloat16]
    y = ops.gated_conv_step(u[:, L], state, w)
    longer = ops.gated_conv_prefill(u, w)
    assert rel_err(y.float(), longer[:, L].float()) < 1e-2
    assert torch.equal(longer[:, :L], v)
