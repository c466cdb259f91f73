"""The drop-in mixers on the GPU against golden vectors of the reference's own modules and
against the CPU oracle."""
import pytest
import torch

from conftest import load_golden, rel_err
from oracle import based_oracle as O

pytestmark = pytest.mark.gpu


def _load_linattn(g, dtype):
    from based_b200.mixers import LinearAttention, TaylorExp
    d_model, H, d, dv, B, L, steps = [int(x) for x in g["meta"]]
    m = LinearAttention(d_model=d_model, feature_map=TaylorExp(input_dim=d), feature_dim=d, num_heads=H,
                        head_dim=dv, layer_idx=0)
    m.load_state_dict({"proj_q.weight": g["wq"], "proj_k.weight": g["wk"], "proj_v.weight": g["wv"],
                       "out_proj.weight": g["wo"]})
    return m.to("cuda", dtype), (d_model, H, d, dv, B, L, steps)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 3e-2)])
def test_linear_attention_mixer_vs_reference_golden(dtype, tol):
    """forward (training path), prefill + decode through InferenceParams: outputs and states
    the reference's LinearAttention produced with the same weights and inputs (fp32)."""
    from based_b200.generation import InferenceParams
    g = load_golden("linattn_mixer.npz")
    m, (d_model, H, d, dv, B, L, steps) = _load_linattn(g, dtype)
    x = g["x"].to("cuda", dtype)
    with torch.inference_mode():
        y_train = m(x[:, :L])
        ip = InferenceParams(max_seqlen=L + steps, max_batch_size=B)
        y_prefill = m(x[:, :L], inference_params=ip)
        kv, ks = ip.key_value_memory_dict[0]
        assert kv.shape == (B, H, 1, dv, 273) and ks.shape == (B, H, 1, 1, 273) and kv.dtype == dtype
        assert rel_err(y_train.float().cpu(), g["y_train"]) < tol
        assert rel_err(y_prefill.float().cpu(), g["y_prefill"]) < tol
        assert rel_err(kv.float().cpu(), g["kv_state_prefill"]) < tol
        assert rel_err(ks.float().cpu(), g["k_state_prefill"]) < tol
        for s in range(steps):
            ip.seqlen_offset = L + s
            y = m(x[:, L + s:L + s + 1], inference_params=ip)
            assert y.shape == (B, 1, d_model)
            assert rel_err(y.float().cpu(), g["y_decode"][:, s:s + 1]) < tol
        assert ip.key_value_memory_dict[0][0] is kv  # updated in place
        assert rel_err(kv.float().cpu(), g["kv_state_final"]) < tol


def test_linear_attention_preallocated_cache_is_filled_in_place():
    """The CUDA-graph flow of the reference (generation.py:629-643): the cache is allocated
    first, prefill must fill those very tensors."""
    from based_b200.generation import InferenceParams
    g = load_golden("linattn_mixer.npz")
    m, (d_model, H, d, dv, B, L, steps) = _load_linattn(g, torch.float32)
    ip = InferenceParams(max_seqlen=L + steps, max_batch_size=B)
    ip.key_value_memory_dict[0] = m.allocate_inference_cache(B, L + steps, dtype=torch.float32)
    kv, ks = ip.key_value_memory_dict[0]
    with torch.inference_mode():
        m(g["x"][:, :L].cuda(), inference_params=ip)
    assert rel_err(kv.cpu(), g["kv_state_prefill"]) < 1e-4 and rel_err(ks.cpu(), g["k_state_prefill"]) < 1e-4


def test_linear_attention_config1_against_reference_samples():
    """The parity configuration at full size (d_model 1024, 16 heads, B=2, L=1024, fp32, seed 0)."""
    from based_b200.generation import InferenceParams
    from based_b200.mixers import LinearAttention, TaylorExp
    g = load_golden("linattn_config1_samples.npz")
    torch.manual_seed(0)
    m = LinearAttention(d_model=1024, feature_map=TaylorExp(input_dim=16), feature_dim=16, num_heads=16,
                        head_dim=64, layer_idx=0)
    x = torch.randn(2, 1024, 1024)
    if rel_err(x[:, ::301, ::307], g["x_probe"]) > 0 or rel_err(m.proj_q.weight[::31, ::101], g["wq_probe"]) > 0:
        pytest.skip("torch RNG stream differs from the one the fixture was generated with")
    m = m.cuda()
    ip = InferenceParams(max_seqlen=1024, max_batch_size=2)
    with torch.inference_mode():
        y = m(x.cuda(), inference_params=ip)
    kv, ks = ip.key_value_memory_dict[0]
    assert rel_err(y[:, ::37, ::29].cpu(), g["y"]) < 1e-4
    assert rel_err(kv[:, ::5, :, ::7, ::11].cpu(), g["kv_state"]) < 1e-4
    assert rel_err(ks[..., ::3].cpu(), g["k_state"]) < 1e-4


def _swa_oracle(x, wqkv, wo, H, hd, w, cos, sin, offset=0):
    B, L, _ = x.shape
    qkv = (x @ wqkv.T).bfloat16().view(B, L, 3, H, hd)
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    if cos is not None:
        q, k = O.apply_rotary(q, cos, sin, offset), O.apply_rotary(k, cos, sin, offset)
    ctx = O.swa_prefill(q.double(), k.double(), v.double(), w).bfloat16()
    return (ctx.reshape(B, L, H * hd).to(x.dtype) @ wo.T), k, v


@pytest.mark.parametrize("rotary", [True, False])
def test_sliding_attention_mixer_prefill_and_decode(rotary):
    from based_b200.generation import InferenceParams
    from based_b200.mixers import SlidingAttention
    torch.manual_seed(1)
    D, H, B, L, N = 256, 4, 2, 100, 5
    hd = D // H
    m = SlidingAttention(D, H, qkv_proj_bias=False, out_proj_bias=False, layer_idx=1, window_size=128,
                         rotary_emb_dim=hd if rotary else 0, dtype=torch.bfloat16).cuda()
    x = torch.randn(B, L + N, D).bfloat16()
    wqkv, wo = m.Wqkv.weight.detach().cpu(), m.out_proj.weight.detach().cpu()
    cos = sin = None
    if rotary:
        cos, sin = O.rotary_cos_sin(L + N, hd, dtype=torch.bfloat16)
    ref_full, _, _ = _swa_oracle(x.float(), wqkv.float(), wo.float(), H, hd, 64, cos, sin)
    with torch.inference_mode():
        y_train = m(x[:, :L].cuda())
        assert rel_err(y_train.float().cpu(), ref_full[:, :L]) < 3e-2
        ip = InferenceParams(max_seqlen=L + N, max_batch_size=B)
        y_pre = m(x[:, :L].cuda(), inference_params=ip)
        assert rel_err(y_pre.float().cpu(), ref_full[:, :L]) < 3e-2
        assert ip.key_value_memory_dict[1].shape == (B, L + N, 2, H, hd)
        for s in range(N):  # decode over the cache == the full-length parallel answer
            ip.seqlen_offset = L + s
            y = m(x[:, L + s:L + s + 1].cuda(), inference_params=ip)
            assert rel_err(y.float().cpu(), ref_full[:, L + s:L + s + 1]) < 3e-2, s


def test_linear_attention_fused_qkv_projection_is_the_same_mixer():
    """One GEMM over the concatenated projection weights: same outputs and states, prompt pass and steps;
    a later change of a projection weight is picked up."""
    import copy
    from based_b200.generation import InferenceParams
    from based_b200.mixers import LinearAttention, TaylorExp
    torch.manual_seed(3)
    a = LinearAttention(256, feature_map=TaylorExp(input_dim=16), num_heads=4, layer_idx=0).to("cuda", torch.bfloat16).eval()
    b = copy.deepcopy(a)
    b.fuse_qkv = True
    x = torch.randn(2, 200, 256, device="cuda", dtype=torch.bfloat16)
    with torch.inference_mode():
        ia, ib = InferenceParams(max_seqlen=256, max_batch_size=2), InferenceParams(max_seqlen=256, max_batch_size=2)
        ya, yb = a(x, inference_params=ia), b(x, inference_params=ib)
        assert torch.equal(ya, yb)
        assert torch.equal(ia.key_value_memory_dict[0][0], ib.key_value_memory_dict[0][0])
        ia.seqlen_offset = ib.seqlen_offset = 200
        xt = torch.randn(2, 1, 256, device="cuda", dtype=torch.bfloat16)
        assert torch.allclose(a(xt, inference_params=ia).float(), b(xt, inference_params=ib).float(), atol=2e-2, rtol=2e-2)
        b.proj_v.weight.mul_(2.0)
        a.proj_v.weight.mul_(2.0)
        assert torch.equal(a(x), b(x))


def test_mixers_refuse_autograd_instead_of_dropping_gradients():
    """The kernels have no backward.  Under grad mode a call must raise — not return an output cut off from the graph,
    which would leave the projections in front of the kernel without gradients and say nothing."""
    from based_b200 import ops
    from based_b200.mixers import BaseConv, LinearAttention, SlidingAttention, TaylorExp
    from based_b200.modules import GatedMlp, RMSNorm
    torch.manual_seed(0)
    x = torch.randn(2, 24, 64, device="cuda", dtype=torch.bfloat16)
    mods = [LinearAttention(64, feature_map=TaylorExp(16), num_heads=2, head_dim=32),
            SlidingAttention(64, 2, qkv_proj_bias=False, out_proj_bias=False, window_size=64),
            BaseConv(64, l_max=64, kernel_size=3), RMSNorm(64), GatedMlp(64, activation=torch.nn.functional.silu)]
    for m in mods:
        m = m.to("cuda", torch.bfloat16)
        with pytest.raises(RuntimeError, match="inference-only"):
            m(x.clone().requires_grad_())
        with pytest.raises(RuntimeError, match="inference-only"):
            m(x)                                    # the parameters require grad
        with torch.inference_mode():
            assert m(x).shape == x.shape
        with torch.no_grad():
            assert m(x).shape == x.shape
    q = torch.randn(1, 2, 8, 16, device="cuda").requires_grad_()
    v = torch.randn(1, 2, 8, 32, device="cuda")
    with pytest.raises(RuntimeError, match="inference-only"):
        ops.linattn_prefill(q, q, v)
    y, _, _ = ops.linattn_prefill(q.detach(), q.detach(), v)
    assert y.shape == (1, 2, 8, 32)
