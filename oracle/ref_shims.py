"""Import the reference's own modules from a staged copy (TEST INFRASTRUCTURE, not product code).

``reference()`` puts ``oracle/_ref`` (see ``oracle/make_ref.py``; or another root given
explicitly) on ``sys.path``, installs the four stand-ins this image needs, imports the
reference's ``based`` package and returns its pieces.  None of the stand-ins touches the
arithmetic that tests pin:

1. ``transformers.generation.GreedySearchDecoderOnlyOutput`` / ``SampleDecoderOnlyOutput``:
   based/generation.py:15 imports them, newer ``transformers`` no longer exports them.  A plain
   attribute bag takes their place (``decode`` only builds one and reads its fields,
   generation.py:203-204, :574-577).
2. ``hydra.utils.instantiate``: hydra is not installed; based/models/gpt.py:90-96 needs
   ``_target_`` / ``_partial_`` resolution of nested dicts and nothing else.
3. ``based.ops.triton.layer_norm.rms_norm_fn`` -> the reference's own ``rms_norm_ref``
   (layer_norm.py:74-125), the Triton kernel's stated semantics; the Triton kernel needs a GPU
   and Triton is not allowed near the product path.
4. ``based.models.mlp.swiglu = None`` so that ``GatedMlp`` takes its torch branch
   (mlp.py:146-153) instead of flash-attn's jiterator op.
"""
import contextlib
import functools
import importlib
import io
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_ROOT = os.path.join(HERE, "_ref")

_cached = None


def _instantiate(cfg, *args, _partial_=False, **kwargs):
    """The subset of ``hydra.utils.instantiate`` that gpt.py:90-96 uses."""
    cfg = dict(cfg)
    partial = cfg.pop("_partial_", _partial_)
    mod, _, attr = cfg.pop("_target_").rpartition(".")
    target = getattr(importlib.import_module(mod), attr)
    cfg.pop("_recursive_", None)
    built = {k: (_instantiate(v) if isinstance(v, dict) and "_target_" in v else v) for k, v in cfg.items()}
    built.update(kwargs)
    return functools.partial(target, *args, **built) if partial else target(*args, **built)


def available(root: str = None) -> bool:
    root = root or DEFAULT_ROOT
    return os.path.exists(os.path.join(root, "based", "models", "mixers", "linear_attention.py"))


def reference(root: str = None, model: bool = True):
    """Namespace with the reference's ``LinearAttention``, ``TaylorExp``, ``InferenceParams`` and, with
    ``model``, ``BaseConv``, ``GPTLMHeadModel``, ``GPT2MixerConfig``, ``rms_norm_ref`` and, where flash-attn
    imports, ``SlidingAttention`` (else None).  Raises FileNotFoundError when nothing is staged."""
    global _cached
    root = root or DEFAULT_ROOT
    if _cached is not None and _cached.root == root and (_cached.model or not model):
        return _cached
    if not available(root):
        raise FileNotFoundError(f"no staged reference under {root}: run `python oracle/make_ref.py --ref <tree>`")
    import transformers.generation as tg

    for name in ("GreedySearchDecoderOnlyOutput", "SampleDecoderOnlyOutput"):
        if not hasattr(tg, name):
            setattr(tg, name, types.SimpleNamespace)
    if "hydra" not in sys.modules:
        hydra = types.ModuleType("hydra")
        hydra.utils = types.ModuleType("hydra.utils")
        hydra.utils.instantiate = _instantiate
        sys.modules["hydra"] = hydra
        sys.modules["hydra.utils"] = hydra.utils
    if root not in sys.path:
        sys.path.insert(0, root)
    ns = types.SimpleNamespace(root=root, model=model)
    with contextlib.redirect_stdout(io.StringIO()):   # the reference prints at import time
        from based.generation import InferenceParams
        from based.models.mixers.linear_attention import LinearAttention, TaylorExp
        ns.InferenceParams, ns.LinearAttention, ns.TaylorExp = InferenceParams, LinearAttention, TaylorExp
        if model:
            import based.models.mlp as mlp
            import based.ops.triton.layer_norm as ln

            def rms_norm_fn(x, weight, bias, residual=None, eps=1e-6, dropout_p=0.0, prenorm=False,
                            residual_in_fp32=False, **kw):
                return ln.rms_norm_ref(x, weight, bias, residual=residual, eps=eps, prenorm=prenorm, upcast=True)

            ln.rms_norm_fn = rms_norm_fn
            mlp.swiglu = None
            from based.models.gpt import GPT2MixerConfig, GPTLMHeadModel
            from based.models.mixers.convolution import BaseConv
            ns.GPT2MixerConfig, ns.GPTLMHeadModel, ns.BaseConv = GPT2MixerConfig, GPTLMHeadModel, BaseConv
            ns.rms_norm_ref, ns.GatedMlp = ln.rms_norm_ref, mlp.GatedMlp
            try:
                from based.models.mixers.slide_attention import SlidingAttention
                ns.SlidingAttention = SlidingAttention
            except Exception:  # flash-attn missing or not importable on this machine
                ns.SlidingAttention = None
    _cached = ns
    return ns


def based_config(ns, *, n_embd, n_layer, n_head, n_inner, vocab_size, alt_mixer_layers, alt_mixer_2_layers,
                 l_max, window_size=128, targets="reference"):
    """A ``GPT2MixerConfig`` of the Based layout (train/configs/experiment/reference/based-360m.yaml:49-117) with the
    mixer ``_target_`` paths pointing at the reference's classes (``targets="reference"``) or at ``based_b200``'s."""
    if targets == "reference":
        conv, lin, fmap, slide = ("based.models.mixers.convolution.BaseConv",
                                  "based.models.mixers.linear_attention.LinearAttention",
                                  "based.models.mixers.linear_attention.TaylorExp",
                                  "based.models.mixers.slide_attention.SlidingAttention")
    else:
        conv, lin, fmap, slide = ("based_b200.mixers.convolution.BaseConv",
                                  "based_b200.mixers.linear_attention.LinearAttention",
                                  "based_b200.mixers.linear_attention.TaylorExp",
                                  "based_b200.mixers.slide_attention.SlidingAttention")
    return ns.GPT2MixerConfig(
        n_embd=n_embd, n_layer=n_layer, n_head=n_head, n_inner=n_inner, vocab_size=vocab_size, n_positions=0,
        max_position_embeddings=0,
        mixer={"_target_": conv, "l_max": l_max, "use_bias": True, "expand_proj": 4, "kernel_size": 3},
        alt_mixer={"_target_": lin, "l_max": l_max, "feature_map": {"_target_": fmap, "input_dim": 16},
                   "feature_dim": 16, "num_heads": n_head, "parallel_implementation": "quadratic"},
        alt_mixer_2={"_target_": slide, "window_size": window_size, "num_heads": n_head, "causal": True},
        alt_mixer_layers=list(alt_mixer_layers), alt_mixer_2_layers=list(alt_mixer_2_layers),
        rms_norm=True, fused_mlp=False, attn_pdrop=0, embd_pdrop=0, resid_pdrop=0, mlp_fc1_bias=False,
        mlp_fc2_bias=False, fused_bias_fc=False, out_proj_bias=False, qkv_proj_bias=False, use_flash_attn=True,
        residual_in_fp32=True, activation_function="swiglu", rotary_emb_fraction=1, fused_dropout_add_ln=False,
        pad_vocab_size_multiple=8, special_initializer=True, fixed_decay=False)
