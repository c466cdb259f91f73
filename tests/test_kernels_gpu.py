"""Parity of the CUDA kernels (called through the C ABI) with the CPU oracle and with the
golden vectors the reference produced.  Tolerances: relative error (max |a-b| / max |b|)
1e-4 for fp32 I/O and 2e-2 for bf16 I/O, against an fp64/fp32 oracle on the same inputs."""
import pytest
import torch

from conftest import load_golden, rel_err, state_block_errs, worst_window_err
from oracle import based_oracle as O

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2}


@pytest.fixture(scope="module")
def ops():
    from based_b200 import ops as _ops
    return _ops


def _qkv(B, H, L, dv, dtype, seed=0, qscale=0.5):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, H, L, 16, generator=g) * qscale).to(dtype)
    k = (torch.randn(B, H, L, 16, generator=g) * qscale).to(dtype)
    v = torch.randn(B, H, L, dv, generator=g).to(dtype)
    return q, k, v


# ------------------------------------------------------------------ linear attention prefill
@pytest.mark.parametrize("impl", ["simt", "tcgen05"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("L,dv", [(1, 64), (15, 64), (16, 64), (17, 64), (77, 64), (128, 64), (129, 64), (300, 112),
                                  (1024, 64), (130, 128), (64, 16)])
def test_linattn_prefill_vs_oracle(ops, impl, dtype, L, dv):
    if impl == "tcgen05" and dtype == torch.float32:
        pytest.skip("the tensor-core kernel takes bf16 I/O only")
    B, H = 2, 3
    q, k, v = _qkv(B, H, L, dv, dtype, seed=L + dv)
    if impl == "tcgen05" and dv > 112:
        from based_b200._capi import BasedLibraryError
        with pytest.raises(BasedLibraryError):  # V' = dv + 16 columns must fit 128 TMEM lanes
            ops.linattn_prefill(q.cuda(), k.cuda(), v.cuda(), impl=impl)
        return
    y_ref, kv_ref, ks_ref = O.linattn_chunked(q.double(), k.double(), v.double(), chunk=128)
    y, kv, ks = ops.linattn_prefill(q.cuda(), k.cuda(), v.cuda(), impl=impl, state_dtype=torch.float32)
    torch.cuda.synchronize()
    from based_b200 import _capi
    assert _capi.read_status() == 0
    tol = TOL[dtype]
    assert y.shape == (B, H, L, dv) and kv.shape == (B, H, 1, dv, 273) and ks.shape == (B, H, 1, 1, 273)
    assert rel_err(y.cpu(), y_ref) < tol
    assert rel_err(kv.cpu(), kv_ref) < tol
    assert rel_err(ks.cpu(), ks_ref) < tol
    # late rows and the small second-order blocks of the state, each against its own scale
    assert worst_window_err(y.cpu(), y_ref, 2, length=32) < tol
    for name, e in {**state_block_errs(kv.cpu(), kv_ref), **{"k_" + n: e for n, e in state_block_errs(ks.cpu(), ks_ref).items()}}.items():
        assert e < tol, (name, e)


@pytest.mark.parametrize("B,H,L,dv,nseg", [(1, 2, 1024, 64, 2), (1, 2, 1024 + 77, 64, 3), (2, 1, 4096, 64, 8),
                                            (1, 1, 2048, 32, 4), (1, 1, 2048 + 5, 112, 5), (1, 3, 300, 64, 64),
                                            (1, 1, 128, 64, 4)])
def test_linattn_prefill_sequence_split_vs_oracle(ops, B, H, L, dv, nseg):
    """The sequence-split form (three launches) against the oracle and the single-launch kernel."""
    from based_b200 import _capi
    q, k, v = _qkv(B, H, L, dv, torch.bfloat16, seed=L + dv + nseg)
    y_ref, kv_ref, ks_ref = O.linattn_chunked(q.double(), k.double(), v.double(), chunk=128)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    y, kv, ks = ops.linattn_prefill(qc, kc, vc, state_dtype=torch.float32, nseg=nseg)
    y1, kv1, ks1 = ops.linattn_prefill(qc, kc, vc, state_dtype=torch.float32, nseg=1)
    torch.cuda.synchronize()
    assert _capi.read_status() == 0
    tol = TOL[torch.bfloat16]
    assert rel_err(y.cpu(), y_ref) < tol
    assert rel_err(kv.cpu(), kv_ref) < tol
    assert rel_err(ks.cpu(), ks_ref) < tol
    assert worst_window_err(y.cpu(), y_ref, 2) < tol
    for name, e in state_block_errs(kv.cpu(), kv_ref).items():
        assert e < tol, (name, e)
    # the split only changes the order of fp32 additions in the state
    assert rel_err(y.float(), y1.float()) < 1e-2
    assert rel_err(kv, kv1) < 1e-5
    # outputs only, no state requested
    y2, none_kv, none_ks = ops.linattn_prefill(qc, kc, vc, return_state=False, nseg=nseg)
    assert none_kv is None and none_ks is None
    assert torch.equal(y2, y)


def test_linattn_prefill_split_chosen_by_library_and_workspace_checks(ops):
    from based_b200 import _capi
    lib = _capi.lib()
    B, H, L, dv = 1, 2, 8192, 64
    auto = lib.based_linattn_prefill_segments(B, H, L)
    assert auto > 1                                     # two (batch, head) pairs leave the machine idle
    assert lib.based_linattn_prefill_segments(64, 16, L) == 1
    assert lib.based_linattn_prefill_segments(B, H, 512) == 1
    need = lib.based_linattn_prefill_scratch_bytes(B, H, L, dv, auto)
    assert need > 0 and lib.based_linattn_prefill_scratch_bytes(B, H, L, dv, 1) == 0
    q, k, v = _qkv(B, H, L, dv, torch.bfloat16, seed=11)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    y_auto, kv_auto, _ = ops.linattn_prefill(qc, kc, vc, state_dtype=torch.float32)          # library's choice
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    y_ws, kv_ws, _ = ops.linattn_prefill(qc, kc, vc, state_dtype=torch.float32, nseg=auto, scratch=ws)
    assert torch.equal(y_auto, y_ws) and torch.equal(kv_auto, kv_ws)
    y_ref, kv_ref, _ = O.linattn_chunked(q.double(), k.double(), v.double(), chunk=128)
    assert rel_err(y_auto.cpu(), y_ref) < TOL[torch.bfloat16]
    assert rel_err(kv_auto.cpu(), kv_ref) < TOL[torch.bfloat16]
    with pytest.raises(_capi.BasedLibraryError):        # workspace one byte short
        ops.linattn_prefill(qc, kc, vc, nseg=auto, scratch=ws[: need - 16])
    with pytest.raises(ValueError):                     # fp32 I/O has no split form
        ops.linattn_prefill(qc.float(), kc.float(), vc.float(), nseg=2)
    torch.cuda.synchronize()
    assert _capi.read_status() == 0


def test_linattn_prefill_golden_fp32(ops):
    """Golden vectors the reference itself produced (quadratic branch, fp64 run)."""
    g = load_golden("linattn_qkv_f64.npz")
    L = g["y_prefill"].shape[1]
    B, H = g["q"].shape[:2]
    q, k, v = (g[n][:, :, :L].float().cuda() for n in ("q", "k", "v"))
    y, kv, ks = ops.linattn_prefill(q, k, v)
    y = y.permute(0, 2, 1, 3).reshape(B, L, -1)
    assert rel_err(y.cpu(), g["y_prefill"]) < 1e-4
    assert rel_err(kv.cpu(), g["kv_state_prefill"]) < 1e-4
    assert rel_err(ks.cpu(), g["k_state_prefill"]) < 1e-4


def test_linattn_prefill_strided_views_and_no_state(ops):
    """q/k/v as the transposed views LinearAttention.forward makes (linear_attention.py:127-129)."""
    B, L, H, dv = 2, 50, 4, 64
    torch.manual_seed(5)
    qf, kf, vf = torch.randn(B, L, H * 16) / 2, torch.randn(B, L, H * 16) / 2, torch.randn(B, L, H * dv)
    q = qf.cuda().view(B, L, H, 16).transpose(1, 2)
    k = kf.cuda().view(B, L, H, 16).transpose(1, 2)
    v = vf.cuda().view(B, L, H, dv).transpose(1, 2)
    y, kv, ks = ops.linattn_prefill(q, k, v, return_state=False)
    assert kv is None and ks is None
    y_ref, _, _ = O.linattn_parallel(q.cpu().double(), k.cpu().double(), v.cpu().double())
    assert rel_err(y.cpu(), y_ref) < 1e-4
    assert y.permute(0, 2, 1, 3).is_contiguous()  # the 'b h l d -> b l (h d)' rearrange is free


def test_linattn_prefill_empty_sequence(ops):
    q = torch.zeros(1, 2, 0, 16, device="cuda")
    v = torch.zeros(1, 2, 0, 64, device="cuda")
    y, kv, ks = ops.linattn_prefill(q, q, v)
    assert y.shape == (1, 2, 0, 64) and kv.abs().max() == 0 and ks.abs().max() == 0


# ------------------------------------------------------------------ linear attention decode
@pytest.mark.parametrize("io,st", [(torch.bfloat16, torch.float32), (torch.float32, torch.float32),
                                   (torch.bfloat16, torch.bfloat16), (torch.float32, torch.bfloat16)])
@pytest.mark.parametrize("dv", [64, 112, 16])
def test_linattn_decode_vs_oracle(ops, io, st, dv):
    B, H, steps = 3, 5, 4
    g = torch.Generator().manual_seed(dv)
    kv0 = (0.02 * torch.randn(B, H, 1, dv, 273, generator=g)).to(st)
    ks0 = (1.0 + 0.02 * torch.randn(B, H, 1, 1, 273, generator=g)).to(st)
    kv_ref, ks_ref = kv0.double(), ks0.double()
    kv, ks = kv0.cuda(), ks0.cuda()
    tol = 2e-2 if (io == torch.bfloat16 or st == torch.bfloat16) else 1e-4
    for s in range(steps):
        q = (torch.randn(B, H, 1, 16, generator=g) / 2).to(io)
        k = (torch.randn(B, H, 1, 16, generator=g) / 2).to(io)
        v = torch.randn(B, H, 1, dv, generator=g).to(io)
        y_ref = O.linattn_recurrent_step(kv_ref, ks_ref, q.double(), k.double(), v.double())
        y = ops.linattn_decode(q.cuda(), k.cuda(), v.cuda(), kv, ks)
        assert y.shape == (B, 1, H * dv) and y.dtype == io
        y_ref = y_ref.transpose(1, 2).reshape(B, 1, H * dv)
        assert rel_err(y.cpu(), y_ref) < tol, f"step {s}"
        assert rel_err(kv.cpu(), kv_ref) < tol and rel_err(ks.cpu(), ks_ref) < tol
        if st == torch.bfloat16:
            # the oracle follows the state as stored (bf16), like the reference does
            kv_ref, ks_ref = kv.cpu().double(), ks.cpu().double()


@pytest.mark.parametrize("io,st,B,H,dv", [(torch.bfloat16, torch.float32, 19, 16, 64), (torch.float32, torch.float32, 37, 8, 32),
                                          (torch.bfloat16, torch.bfloat16, 40, 8, 16), (torch.bfloat16, torch.float32, 20, 16, 112),
                                          (torch.bfloat16, torch.float32, 75, 4, 64)])
def test_linattn_decode_many_heads_vs_oracle(ops, io, st, B, H, dv):
    """More (batch, head) blocks than SMs x resident CTAs, several head counts and widths, three steps each."""
    from based_b200 import _capi
    g = torch.Generator().manual_seed(B + dv)
    kv0 = (0.02 * torch.randn(B, H, 1, dv, 273, generator=g)).to(st)
    ks0 = (1.0 + 0.02 * torch.randn(B, H, 1, 1, 273, generator=g)).to(st)
    kv_ref, ks_ref = kv0.double(), ks0.double()
    kv, ks = kv0.cuda(), ks0.cuda()
    tol = 2e-2 if (io == torch.bfloat16 or st == torch.bfloat16) else 1e-4
    for s in range(3):
        q = (torch.randn(B, H, 1, 16, generator=g) / 2).to(io)
        k = (torch.randn(B, H, 1, 16, generator=g) / 2).to(io)
        v = torch.randn(B, H, 1, dv, generator=g).to(io)
        y_ref = O.linattn_recurrent_step(kv_ref, ks_ref, q.double(), k.double(), v.double())
        y = ops.linattn_decode(q.cuda(), k.cuda(), v.cuda(), kv, ks)
        y_ref = y_ref.transpose(1, 2).reshape(B, 1, H * dv)
        assert rel_err(y.cpu(), y_ref) < tol, f"step {s}"
        assert rel_err(kv.cpu(), kv_ref) < tol and rel_err(ks.cpu(), ks_ref) < tol
        if st == torch.bfloat16:
            kv_ref, ks_ref = kv.cpu().double(), ks.cpu().double()
    torch.cuda.synchronize()
    assert _capi.read_status() == 0


def test_linattn_decode_golden(ops):
    """Decode steps the reference itself ran (recurrent_forward), from its prefill state."""
    g = load_golden("linattn_qkv_f32_dv112.npz")
    L = g["y_prefill"].shape[1]
    B, H, Ltot, _ = g["q"].shape
    kv, ks = g["kv_state_prefill"].cuda().contiguous(), g["k_state_prefill"].cuda().contiguous()
    for s in range(Ltot - L):
        sl = slice(L + s, L + s + 1)
        y = ops.linattn_decode(g["q"][:, :, sl].cuda(), g["k"][:, :, sl].cuda(), g["v"][:, :, sl].cuda(), kv, ks)
        assert rel_err(y.cpu(), g["y_decode"][s]) < 1e-4
    assert rel_err(kv.cpu(), g["kv_state_final"]) < 1e-4
    assert rel_err(ks.cpu(), g["k_state_final"]) < 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prefill_then_decode_equals_longer_prefill(ops, dtype):
    """The reference's own pin (based/tests/test_generation.py:169-173): recurrent == parallel."""
    B, H, L, N, dv = 2, 4, 96, 8, 64
    q, k, v = _qkv(B, H, L + N, dv, dtype, seed=11)
    q, k, v = q.cuda(), k.cuda(), v.cuda()
    y_full, kv_full, ks_full = ops.linattn_prefill(q, k, v, state_dtype=torch.float32)
    _, kv, ks = ops.linattn_prefill(q[:, :, :L], k[:, :, :L], v[:, :, :L], state_dtype=torch.float32)
    tol = TOL[dtype]
    for s in range(N):
        sl = slice(L + s, L + s + 1)
        y = ops.linattn_decode(q[:, :, sl], k[:, :, sl], v[:, :, sl], kv, ks).view(B, H, dv)
        assert rel_err(y.float().cpu(), y_full[:, :, L + s].float().cpu()) < tol
    assert rel_err(kv.cpu(), kv_full.cpu()) < tol and rel_err(ks.cpu(), ks_full.cpu()) < tol


# ------------------------------------------------------------------ sliding-window attention
@pytest.mark.parametrize("impl", ["simt", "tcgen05"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("L,hd,w", [(1, 64, 64), (5, 64, 64), (64, 64, 64), (65, 64, 64), (130, 64, 64),
                                    (300, 112, 64), (257, 64, 128), (200, 128, 0), (1000, 64, 64)])
def test_swa_prefill_vs_oracle(ops, impl, dtype, L, hd, w):
    if impl == "tcgen05" and dtype == torch.float32:
        pytest.skip("the tensor-core kernel takes bf16 I/O only")
    B, H = 2, 3
    g = torch.Generator().manual_seed(L + hd + w)
    qkv = torch.randn(B, L, 3, H, hd, generator=g).to(dtype)
    ref = O.swa_prefill(qkv[:, :, 0].double(), qkv[:, :, 1].double(), qkv[:, :, 2].double(), w)
    qkv_d = qkv.cuda()
    out = ops.swa_prefill(qkv_d[:, :, 0], qkv_d[:, :, 1], qkv_d[:, :, 2], w, impl=impl)
    assert out.shape == (B, L, H, hd) and out.dtype == dtype
    assert rel_err(out.cpu(), ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rotary", [False, True])
@pytest.mark.parametrize("hd", [64, 112])
def test_swa_decode_vs_oracle(ops, dtype, rotary, hd):
    B, H, maxL, w = 3, 4, 100, 64
    g = torch.Generator().manual_seed(hd)
    cache = torch.randn(B, maxL, 2, H, hd, generator=g).to(dtype)
    cache_d = cache.cuda()
    cache_ref = cache.clone()
    cos = sin = cos_d = sin_d = None
    if rotary:
        cos, sin = O.rotary_cos_sin(maxL, hd, dtype=dtype)
        cos_d, sin_d = cos.cuda(), sin.cuda()
    lens = torch.tensor([3, 64, 80], dtype=torch.int32)
    for step in range(5):
        q = torch.randn(B, 1, H, hd, generator=g).to(dtype)
        kn = torch.randn(B, 1, H, hd, generator=g).to(dtype)
        vn = torch.randn(B, 1, H, hd, generator=g).to(dtype)
        ref = O.swa_decode_step(q, kn, vn, cache_ref, lens, w, cos=cos, sin=sin)
        out = ops.swa_decode(q.cuda(), kn.cuda(), vn.cuda(), cache_d, lens.cuda(), w,
                             rotary_cos=cos_d, rotary_sin=sin_d)
        assert rel_err(out.cpu(), ref) < TOL[dtype]
        for b in range(B):  # the appended rows
            p = int(lens[b])
            assert rel_err(cache_d[b, p].cpu(), cache_ref[b, p]) < TOL[dtype]
        lens = lens + 1
    # scalar cache_seqlens path
    q = torch.randn(B, 1, H, hd, generator=g).to(dtype)
    kn, vn = torch.randn(B, 1, H, hd, generator=g).to(dtype), torch.randn(B, 1, H, hd, generator=g).to(dtype)
    ref = O.swa_decode_step(q, kn, vn, cache_ref, 90, w, cos=cos, sin=sin)
    out = ops.swa_decode(q.cuda(), kn.cuda(), vn.cuda(), cache_d, 90, w, rotary_cos=cos_d, rotary_sin=sin_d)
    assert rel_err(out.cpu(), ref) < TOL[dtype]


def test_swa_decode_equals_prefill(ops):
    """Self-consistency the reference's 'sliding' generation test encodes
    (based/tests/test_generation.py:69-80, :169-173): decode over the cache == prefill."""
    B, H, L, N, hd, w = 2, 4, 90, 6, 64, 64
    torch.manual_seed(2)
    qkv = torch.randn(B, L + N, 3, H, hd).bfloat16().cuda()
    full = ops.swa_prefill(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], w)
    cache = torch.zeros(B, L + N, 2, H, hd, dtype=torch.bfloat16, device="cuda")
    cache[:, :L] = qkv[:, :L, 1:]
    for s in range(N):
        t = L + s
        out = ops.swa_decode(qkv[:, t:t + 1, 0], qkv[:, t:t + 1, 1], qkv[:, t:t + 1, 2], cache, t, w)
        assert rel_err(out[:, 0].float().cpu(), full[:, t].float().cpu()) < 2e-2


# ------------------------------------------------------------------ full-size, size-independent properties
def test_prefill_full_size_properties(ops):
    """Prefill-sweep shape (B=8, H=16, L=8192, dv=64, bf16), too large for the quadratic oracle
    as a whole: (1) sampled (batch, head) slices against the chunked fp64 oracle, (2) linearity in v
    (the normaliser does not depend on v), (3) recurrent == parallel for the last positions,
    (4) tensor-core and CUDA-core kernels agree."""
    B, H, L, dv = 8, 16, 8192, 64
    g = torch.Generator(device="cuda").manual_seed(0)
    q = (torch.randn(B, H, L, 16, device="cuda", generator=g) / 4).bfloat16()
    k = (torch.randn(B, H, L, 16, device="cuda", generator=g) / 4).bfloat16()
    v1 = (torch.randn(B, H, L, dv, device="cuda", generator=g) / 4).bfloat16()
    v2 = (torch.randn(B, H, L, dv, device="cuda", generator=g) / 4).bfloat16()
    y1, kv1, ks1 = ops.linattn_prefill(q, k, v1, state_dtype=torch.float32)
    y2, kv2, ks2 = ops.linattn_prefill(q, k, v2, state_dtype=torch.float32)
    v12 = (v1.float() + v2.float()).bfloat16()
    y12, kv12, _ = ops.linattn_prefill(q, k, v12, state_dtype=torch.float32)
    from based_b200 import _capi
    assert _capi.read_status() == 0
    # (1) sampled slices vs the oracle
    for (b, h) in [(0, 0), (3, 7), (7, 15)]:
        yr, kvr, ksr = O.linattn_chunked(q[b:b + 1, h:h + 1].cpu().double(), k[b:b + 1, h:h + 1].cpu().double(),
                                         v1[b:b + 1, h:h + 1].cpu().double(), chunk=512)
        assert rel_err(y1[b:b + 1, h:h + 1].cpu(), yr) < 2e-2
        assert worst_window_err(y1[b:b + 1, h:h + 1].cpu(), yr, 2) < 2e-2
        for name, e in state_block_errs(kv1[b:b + 1, h:h + 1].cpu(), kvr).items():
            assert e < 2e-2, (b, h, name, e)
        assert rel_err(kv1[b:b + 1, h:h + 1].cpu(), kvr) < 2e-2
        assert rel_err(ks1[b:b + 1, h:h + 1].cpu(), ksr) < 2e-2
    # (2) linearity in v (bf16 rounding of the inputs/outputs bounds the slack)
    assert rel_err(y12.float(), y1.float() + y2.float()) < 2e-2
    assert rel_err(kv12, kv1 + kv2) < 2e-2
    assert torch.equal(ks1, ks2)  # k_state does not depend on v: bit-identical
    # (3) one decode step from the state of the first L-1 tokens reproduces the last prefill row
    _, kvp, ksp = ops.linattn_prefill(q[:, :, :L - 1], k[:, :, :L - 1], v1[:, :, :L - 1], state_dtype=torch.float32)
    yd = ops.linattn_decode(q[:, :, L - 1:], k[:, :, L - 1:], v1[:, :, L - 1:], kvp, ksp).view(B, H, dv)
    assert rel_err(yd.float(), y1[:, :, L - 1].float()) < 2e-2
    assert rel_err(kvp, kv1) < 2e-2
    # (4) the two prefill kernels agree on a slice
    ys, kvs, _ = ops.linattn_prefill(q[:1, :2], k[:1, :2], v1[:1, :2], impl="simt", state_dtype=torch.float32)
    assert rel_err(y1[:1, :2].float(), ys.float()) < 2e-2 and rel_err(kv1[:1, :2], kvs) < 2e-2


def test_decode_full_size_properties(ops):
    """Decode-microbenchmark shape (B=256, H=16, fp32 state): sampled units against the oracle after
    several in-place steps, and determinism (two runs from the same state are bit-identical)."""
    B, H, dv = 256, 16, 64
    g = torch.Generator(device="cuda").manual_seed(1)
    kv0 = 0.02 * torch.randn(B, H, 1, dv, 273, device="cuda", generator=g)
    ks0 = 1.0 + 0.02 * torch.randn(B, H, 1, 1, 273, device="cuda", generator=g)
    steps = 5
    qs = (torch.randn(steps, B, H, 1, 16, device="cuda", generator=g) / 4).bfloat16()
    kk = (torch.randn(steps, B, H, 1, 16, device="cuda", generator=g) / 4).bfloat16()
    vs = torch.randn(steps, B, H, 1, dv, device="cuda", generator=g).bfloat16()
    outs = []
    for run in range(2):
        kv, ks = kv0.clone(), ks0.clone()
        ys = [ops.linattn_decode(qs[s], kk[s], vs[s], kv, ks).clone() for s in range(steps)]
        outs.append((torch.stack(ys), kv, ks))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    idx = [(0, 0), (100, 5), (255, 15)]
    for (b, h) in idx:
        kvr, ksr = kv0[b:b + 1, h:h + 1].cpu().double(), ks0[b:b + 1, h:h + 1].cpu().double()
        for s in range(steps):
            yr = O.linattn_recurrent_step(kvr, ksr, qs[s, b:b + 1, h:h + 1].cpu().double(),
                                          kk[s, b:b + 1, h:h + 1].cpu().double(), vs[s, b:b + 1, h:h + 1].cpu().double())
            got = outs[0][0][s, b, 0, h * dv:(h + 1) * dv].float().cpu()
            assert rel_err(got, yr.flatten()) < 2e-2
        assert rel_err(outs[0][1][b:b + 1, h:h + 1].cpu(), kvr) < 1e-4


def test_swa_full_size_properties(ops):
    """Config-3 sliding-window shape (B=8, L=8192, H=16, hd=64, w=64): sampled heads against the
    oracle; shift invariance (attention over a window depends only on relative positions, so
    dropping the first 128 tokens leaves every row past 128 + w unchanged, bit for bit)."""
    B, L, H, hd, w = 8, 8192, 16, 64, 64
    g = torch.Generator(device="cuda").manual_seed(2)
    qkv = (torch.randn(B, L, 3, H, hd, device="cuda", generator=g) / 4).bfloat16()
    out = ops.swa_prefill(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], w)
    for (b, h) in [(0, 0), (5, 9)]:
        sl = qkv[b:b + 1, :1024, :, h:h + 1].cpu().double()
        ref = O.swa_prefill(sl[:, :, 0], sl[:, :, 1], sl[:, :, 2], w)
        assert rel_err(out[b:b + 1, :1024, h:h + 1].cpu(), ref) < 2e-2
    out_shift = ops.swa_prefill(qkv[:, 128:, 0], qkv[:, 128:, 1], qkv[:, 128:, 2], w)
    assert torch.equal(out_shift[:, w:], out[:, 128 + w:])


def test_decode_step_is_cuda_graph_capturable(ops):
    """The reference replays a captured decode step (based/generation.py:689-739): the kernels must
    launch on the capturing stream, allocate nothing and update the state in place."""
    B, H, dv = 4, 4, 64
    g = torch.Generator(device="cuda").manual_seed(3)
    kv = 0.02 * torch.randn(B, H, 1, dv, 273, device="cuda", generator=g)
    ks = 1.0 + 0.02 * torch.randn(B, H, 1, 1, 273, device="cuda", generator=g)
    kv_ref, ks_ref = kv.clone(), ks.clone()
    q = (torch.randn(B, H, 1, 16, device="cuda", generator=g) / 4).bfloat16()
    k = (torch.randn(B, H, 1, 16, device="cuda", generator=g) / 4).bfloat16()
    v = torch.randn(B, H, 1, dv, device="cuda", generator=g).bfloat16()
    y = torch.empty(B, 1, H * dv, dtype=torch.bfloat16, device="cuda")
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        ops.linattn_decode(q, k, v, kv, ks, out=y)  # warm-up on the side stream
    torch.cuda.current_stream().wait_stream(s)
    kv.copy_(kv_ref); ks.copy_(ks_ref)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ops.linattn_decode(q, k, v, kv, ks, out=y)
    kv.copy_(kv_ref); ks.copy_(ks_ref)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    for _ in range(3):
        y_eager = ops.linattn_decode(q, k, v, kv_ref, ks_ref)
    assert torch.equal(y, y_eager) and torch.equal(kv, kv_ref) and torch.equal(ks, ks_ref)


@pytest.mark.parametrize("B,L,H,hd", [(2, 37, 4, 64), (1, 130, 2, 112), (3, 1, 2, 16)])
def test_rotary_qkv_cache_equals_rotary_then_copy(ops, B, L, H, hd):
    """The fused prompt-pass kernel (RoPE on q, k in place + cache fill) against the separate rotary launches and
    a copy, bit for bit; the oracle pins the rotary itself."""
    g = torch.Generator().manual_seed(hd + L)
    qkv = torch.randn(B, L, 3, H, hd, generator=g).bfloat16()
    cos, sin = O.rotary_cos_sin(L + 9, hd, dtype=torch.bfloat16)
    a, b = qkv.clone().cuda(), qkv.clone().cuda()
    cache = torch.full((B + 1, L + 5, 2, H, hd), 7.0, dtype=torch.bfloat16, device="cuda")
    ops.rotary_qkv_cache_(a, cos.cuda(), sin.cuda(), cache[1:])
    ops.rotary_apply_(b[:, :, 0], cos.cuda(), sin.cuda(), 0)
    ops.rotary_apply_(b[:, :, 1], cos.cuda(), sin.cuda(), 0)
    assert torch.equal(a, b)
    assert torch.equal(cache[1:, :L], b[:, :, 1:])
    assert (cache[0] == 7).all() and (cache[1:, L:] == 7).all()          # nothing else is touched
    ref_q = O.apply_rotary(qkv[:, :, 0], cos, sin, 0)
    assert rel_err(a[:, :, 0].cpu().float(), ref_q.float()) < 1e-2
