"""Generate golden vectors for the linear-attention path from the reference itself.

Run where the HazyResearch/based tree is available (``--ref`` or the
``BASED_REFERENCE`` environment variable points at its root)::

    python tests/golden/make_golden.py --ref /path/to/based

It imports the reference's own ``TaylorExp`` / ``LinearAttention``
(based/models/mixers/linear_attention.py) and ``InferenceParams``
(based/generation.py:18-35) on CPU, runs them on seeded inputs, and writes
small ``.npz`` files next to this script.  The tests never import the
reference; they read these files.

One import shim is needed: based/generation.py:15 imports two output classes
that newer ``transformers`` releases no longer export.
"""
import argparse
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def import_reference(ref_root):
    import transformers.generation as tg

    for name in ("GreedySearchDecoderOnlyOutput", "SampleDecoderOnlyOutput"):
        if not hasattr(tg, name):
            setattr(tg, name, types.SimpleNamespace)
    sys.path.insert(0, ref_root)
    import contextlib
    import io

    with contextlib.redirect_stdout(io.StringIO()):
        from based.generation import InferenceParams
        from based.models.mixers.linear_attention import LinearAttention, TaylorExp
    return LinearAttention, TaylorExp, InferenceParams


def t2n(t):
    # clone: states are updated in place later, and .numpy() would alias them
    return t.detach().to(torch.float64 if t.dtype == torch.float64 else torch.float32).clone().numpy()


def feature_map_case(TaylorExp):
    torch.manual_seed(1)
    x = torch.randn(2, 3, 5, 16, dtype=torch.float64)
    phi = TaylorExp(input_dim=16)(x)
    np.savez(os.path.join(HERE, "taylor_exp.npz"), x=t2n(x), phi=t2n(phi))


def qkv_level_case(LinearAttention, TaylorExp, InferenceParams, name, B, H, L, dv, steps, dtype):
    """Reference prefill on explicit q, k, v (out_proj = identity), then decode steps."""
    torch.manual_seed(7)
    d = 16
    m = LinearAttention(d_model=H * dv, feature_map=TaylorExp(input_dim=d), feature_dim=d,
                        num_heads=H, head_dim=dv).to(dtype)
    m.out_proj = torch.nn.Identity()
    q = (torch.randn(B, H, L + steps, d) / 2).to(dtype)
    k = (torch.randn(B, H, L + steps, d) / 2).to(dtype)
    v = torch.randn(B, H, L + steps, dv).to(dtype)
    x = torch.zeros(B, L, H * dv, dtype=dtype)
    m.is_inference = True
    y, kv_state, k_state = m.parallel_forward(x, q[:, :, :L], k[:, :, :L], v[:, :, :L])
    out = dict(q=t2n(q), k=t2n(k), v=t2n(v), y_prefill=t2n(y),
               kv_state_prefill=t2n(kv_state), k_state_prefill=t2n(k_state))
    kv_state, k_state = kv_state.clone(), k_state.clone()
    fm = m.feature_map
    ys = []
    for s in range(steps):
        sl = slice(L + s, L + s + 1)
        xs = torch.zeros(B, 1, H * dv, dtype=dtype)
        ys.append(m.recurrent_forward(xs, kv_state, k_state, fm(q[:, :, sl]), fm(k[:, :, sl]), v[:, :, sl]))
    out["y_decode"] = t2n(torch.stack(ys, 0))          # [steps, B, 1, H*dv]
    out["kv_state_final"] = t2n(kv_state)
    out["k_state_final"] = t2n(k_state)
    # the full-length parallel answer for the decoded positions (recurrent == parallel pin,
    # based/tests/test_generation.py:169-173)
    m.is_inference = False
    y_full = m.parallel_forward(torch.zeros(B, L + steps, H * dv, dtype=dtype), q, k, v)
    out["y_full"] = t2n(y_full)
    np.savez(os.path.join(HERE, name), **out)


def mixer_level_case(LinearAttention, TaylorExp, InferenceParams):
    """Whole mixer with projections through forward(), prefill + 3 decode steps via InferenceParams."""
    torch.manual_seed(0)
    d_model, H, d, dv, B, L, steps = 64, 2, 16, 32, 2, 37, 3
    m = LinearAttention(d_model=d_model, feature_map=TaylorExp(input_dim=d), feature_dim=d,
                        num_heads=H, head_dim=dv, layer_idx=0)
    x = torch.randn(B, L + steps, d_model)
    y_train = m(x[:, :L])
    ip = InferenceParams(max_seqlen=L + steps, max_batch_size=B)
    y_prefill = m(x[:, :L], inference_params=ip)
    kv0, k0 = [t.clone() for t in ip.key_value_memory_dict[0]]
    ys = []
    for s in range(steps):
        ip.seqlen_offset = L + s
        ys.append(m(x[:, L + s: L + s + 1], inference_params=ip))
    kv1, k1 = ip.key_value_memory_dict[0]
    np.savez(os.path.join(HERE, "linattn_mixer.npz"),
             x=t2n(x), wq=t2n(m.proj_q.weight), wk=t2n(m.proj_k.weight), wv=t2n(m.proj_v.weight),
             wo=t2n(m.out_proj.weight), y_train=t2n(y_train), y_prefill=t2n(y_prefill),
             kv_state_prefill=t2n(kv0), k_state_prefill=t2n(k0),
             y_decode=t2n(torch.cat(ys, 1)), kv_state_final=t2n(kv1), k_state_final=t2n(k1),
             meta=np.array([d_model, H, d, dv, B, L, steps]))


def config1_samples(LinearAttention, TaylorExp, InferenceParams):
    """Parity configuration (d_model 1024, 16 heads, feature_dim 16, head_dim 64, B=2, L=1024, fp32, seed 0):
    the inputs are regenerated from the seed by the test; only strided samples of the outputs are stored."""
    torch.manual_seed(0)
    m = LinearAttention(d_model=1024, feature_map=TaylorExp(input_dim=16), feature_dim=16,
                        num_heads=16, head_dim=64, layer_idx=0)
    x = torch.randn(2, 1024, 1024)
    ip = InferenceParams(max_seqlen=1024, max_batch_size=2)
    with torch.no_grad():
        y = m(x, inference_params=ip)
        y_train = m(x)
    kv, ks = ip.key_value_memory_dict[0]
    np.savez(os.path.join(HERE, "linattn_config1_samples.npz"),
             y=t2n(y[:, ::37, ::29]), y_train=t2n(y_train[:, ::37, ::29]),
             kv_state=t2n(kv[:, ::5, :, ::7, ::11]), k_state=t2n(ks[..., ::3]),
             x_probe=t2n(x[:, ::301, ::307]), wq_probe=t2n(m.proj_q.weight[::31, ::101]),
             y_abs_mean=np.float64(y.abs().mean().item()))


def baseconv_case(ref_root, InferenceParams):
    """Reference BaseConv (based/models/mixers/convolution.py:174-217): train path, prefill with
    state, three decode steps, and a prompt shorter than the kernel."""
    import contextlib
    import io

    with contextlib.redirect_stdout(io.StringIO()):
        from based.models.mixers.convolution import BaseConv
    torch.manual_seed(11)
    d, L, B = 64, 37, 2
    m = BaseConv(d_model=d, l_max=128, kernel_size=3, layer_idx=0).double()
    x = torch.randn(B, L, d, dtype=torch.float64)
    out = {"in_w": t2n(m.in_proj.weight), "in_b": t2n(m.in_proj.bias), "conv_w": t2n(m.conv.conv.weight),
           "out_w": t2n(m.out_proj.weight), "out_b": t2n(m.out_proj.bias), "x": t2n(x)}
    out["y_train"] = t2n(m(x))
    # the op the kernel replaces, isolated: u = in_proj(x) -> v = silu(conv(u1)) * u2
    u = m.in_proj(x)
    u1, u2 = torch.split(u, m.d_inner, dim=-1)
    out["u"] = t2n(u)
    out["v"] = t2n(torch.nn.functional.silu(m.conv(u1)) * u2)
    ip = InferenceParams(max_seqlen=128, max_batch_size=B)
    out["y_prefill"] = t2n(m(x, inference_params=ip))
    out["state_prefill"] = t2n(ip.key_value_memory_dict[0]["conv"])
    for i in range(3):
        ip.seqlen_offset = L + i
        xt = torch.randn(B, 1, d, dtype=torch.float64)
        out[f"x_step{i}"] = t2n(xt)
        out[f"y_step{i}"] = t2n(m(xt, inference_params=ip))
        out[f"state_step{i}"] = t2n(ip.key_value_memory_dict[0]["conv"])
    # prompt of 2 tokens with kernel_size 3: the state keeps a leading zero
    ip2 = InferenceParams(max_seqlen=128, max_batch_size=B)
    xs = torch.randn(B, 2, d, dtype=torch.float64)
    out["x_short"] = t2n(xs)
    out["y_short"] = t2n(m(xs, inference_params=ip2))
    out["state_short"] = t2n(ip2.key_value_memory_dict[0]["conv"])
    np.savez(os.path.join(HERE, "baseconv.npz"), **out)


def norm_mlp_case(ref_root):
    """Reference rms_norm_ref (based/ops/triton/layer_norm.py:74-125) with residual and prenorm, and
    GatedMlp (based/models/mlp.py:99-157) with silu (SwiGLU, torch branch) and sigmoid (GLU)."""
    import contextlib
    import io

    import torch.nn.functional as F

    with contextlib.redirect_stdout(io.StringIO()):
        import based.models.mlp as mlp
        from based.ops.triton.layer_norm import rms_norm_ref
    mlp.swiglu = None  # flash-attn's CUDA op; the torch branch (mlp.py:151-153) states the same mathematics
    torch.manual_seed(13)
    D = 72
    x = torch.randn(3, 7, D, dtype=torch.float64)
    res = torch.randn(3, 7, D, dtype=torch.float64)
    w = torch.randn(D, dtype=torch.float64) * 0.3 + 1.0
    b = torch.randn(D, dtype=torch.float64) * 0.1
    out = {"x": t2n(x), "residual": t2n(res), "weight": t2n(w), "bias": t2n(b)}
    o, r = rms_norm_ref(x, w, None, residual=res, eps=1e-5, prenorm=True)
    out["out_res"], out["res_out"] = t2n(o), t2n(r)
    out["out_nores"] = t2n(rms_norm_ref(x, w, None, eps=1e-5))
    out["out_bias"] = t2n(rms_norm_ref(x, w, b, residual=res, eps=1e-6))
    for name, act in (("silu", F.silu), ("sigmoid", F.sigmoid)):
        m = mlp.GatedMlp(32, activation=act, bias1=False, bias2=False, multiple_of=32).double()
        xm = torch.randn(2, 5, 32, dtype=torch.float64)
        out[f"mlp_{name}_fc1"], out[f"mlp_{name}_fc2"] = t2n(m.fc1.weight), t2n(m.fc2.weight)
        out[f"mlp_{name}_x"], out[f"mlp_{name}_y"] = t2n(xm), t2n(m(xm))
    np.savez(os.path.join(HERE, "norm_mlp.npz"), **out)


def full_model_case(ref_root, InferenceParams):
    """The reference's GPTLMHeadModel (based/models/gpt.py:737-830) on CPU in fp32: BaseConv, LinearAttention
    and BaseConv blocks with RMSNorm and SwiGLU MLPs.  Logits of a full pass, of the prompt pass and of
    three single-token steps, plus the weights.

    Three more shims, none of which touches the arithmetic being pinned: a stand-in for
    ``hydra.utils.instantiate`` (hydra is not installed; gpt.py:90-96 only needs _target_/_partial_
    resolution), ``rms_norm_fn`` -> the reference's own ``rms_norm_ref`` (the Triton kernel needs a GPU;
    layer_norm.py:74-125 is its stated semantics), and ``swiglu = None`` so that GatedMlp takes its torch
    branch (mlp.py:151-153).  The sliding-window mixer cannot run without a GPU and is left out here.
    """
    import contextlib
    import functools
    import importlib
    import io

    def locate(path):
        mod, _, attr = path.rpartition(".")
        return getattr(importlib.import_module(mod), attr)

    def instantiate(cfg, *args, _partial_=False, **kwargs):
        cfg = dict(cfg)
        partial = cfg.pop("_partial_", _partial_)
        target = locate(cfg.pop("_target_"))
        cfg.pop("_recursive_", None)
        built = {k: (instantiate(v) if isinstance(v, dict) and "_target_" in v else v) for k, v in cfg.items()}
        built.update(kwargs)
        return functools.partial(target, *args, **built) if partial else target(*args, **built)

    hydra = types.ModuleType("hydra")
    hydra.utils = types.ModuleType("hydra.utils")
    hydra.utils.instantiate = instantiate
    sys.modules.setdefault("hydra", hydra)
    sys.modules.setdefault("hydra.utils", hydra.utils)
    with contextlib.redirect_stdout(io.StringIO()):
        import based.models.mlp as mlp
        import based.ops.triton.layer_norm as ln

        def rms_norm_fn(x, weight, bias, residual=None, eps=1e-6, dropout_p=0.0, prenorm=False,
                        residual_in_fp32=False, **kw):
            return ln.rms_norm_ref(x, weight, bias, residual=residual, eps=eps, prenorm=prenorm, upcast=True)

        ln.rms_norm_fn = rms_norm_fn
        mlp.swiglu = None
        from based.models.gpt import GPT2MixerConfig, GPTLMHeadModel
    cfg = GPT2MixerConfig(
        n_embd=32, n_layer=3, n_head=2, n_inner=64, vocab_size=97, n_positions=0, max_position_embeddings=0,
        mixer={"_target_": "based.models.mixers.convolution.BaseConv", "l_max": 64, "use_bias": True,
               "expand_proj": 4, "kernel_size": 3},
        alt_mixer={"_target_": "based.models.mixers.linear_attention.LinearAttention", "l_max": 64,
                   "feature_map": {"_target_": "based.models.mixers.linear_attention.TaylorExp", "input_dim": 16},
                   "feature_dim": 16, "num_heads": 2, "parallel_implementation": "quadratic"},
        alt_mixer_layers=[1], alt_mixer_2_layers=[],
        rms_norm=True, fused_mlp=False, attn_pdrop=0, embd_pdrop=0, resid_pdrop=0, mlp_fc1_bias=False,
        mlp_fc2_bias=False, fused_bias_fc=False, out_proj_bias=False, qkv_proj_bias=False, use_flash_attn=False,
        residual_in_fp32=True, activation_function="swiglu", rotary_emb_fraction=1, fused_dropout_add_ln=False,
        pad_vocab_size_multiple=8, special_initializer=True, fixed_decay=False)
    torch.manual_seed(0)
    with contextlib.redirect_stdout(io.StringIO()):
        m = GPTLMHeadModel(cfg)
    # the special initialiser leaves the outputs tiny; scale the weights up so that every layer matters
    with torch.no_grad():
        for name, prm in m.named_parameters():
            if prm.dim() > 1 and "embeddings" not in name:
                prm.mul_(3.0)
    out = {"sd." + k: t2n(v) for k, v in m.state_dict().items() if k != "lm_head.weight"}
    ids = torch.randint(0, 97, (2, 13))
    out["input_ids"] = ids.numpy().copy()
    out["logits_full"] = t2n(m(ids).logits)
    ip = InferenceParams(max_seqlen=32, max_batch_size=2)
    out["logits_prefill_last"] = t2n(m(ids, inference_params=ip, num_last_tokens=1).logits)
    for i in range(3):
        ip.seqlen_offset = 13 + i
        nxt = torch.randint(0, 97, (2, 1))
        out[f"step{i}_ids"] = nxt.numpy().copy()
        out[f"step{i}_logits"] = t2n(m(nxt, inference_params=ip, num_last_tokens=1).logits)
    np.savez(os.path.join(HERE, "full_model.npz"), **out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("BASED_REFERENCE"))
    args = ap.parse_args()
    if not args.ref:
        ap.error("--ref or BASED_REFERENCE must point at the HazyResearch/based tree")
    LA, TE, IP = import_reference(args.ref)
    with torch.no_grad():
        feature_map_case(TE)
        qkv_level_case(LA, TE, IP, "linattn_qkv_f64.npz", B=1, H=2, L=77, dv=64, steps=4, dtype=torch.float64)
        qkv_level_case(LA, TE, IP, "linattn_qkv_f32_dv112.npz", B=1, H=2, L=130, dv=112, steps=2, dtype=torch.float32)
        mixer_level_case(LA, TE, IP)
        config1_samples(LA, TE, IP)
        baseconv_case(args.ref, IP)
        norm_mlp_case(args.ref)
        full_model_case(args.ref, IP)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
