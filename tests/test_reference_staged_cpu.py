"""CPU checks around the staged reference (``oracle/_ref``, built by ``oracle/make_ref.py``):

* the oracle restatement equals the reference's own ``LinearAttention`` run here on the same seeded inputs
  (a direct pin, next to the committed golden vectors);
* the reference's own model factory (based/models/gpt.py:64-145) builds ``based_b200`` mixers from the ``_target_``
  paths that the integration notes give, with the sliding-window additions applied;
* those notes name a sliding-window path that contains ``slide`` (gpt.py:87 keys on that substring).
"""
import os
import re

import pytest
import torch

from conftest import ROOT, rel_err
from oracle import based_oracle as O
from oracle import ref_shims

needs_ref = pytest.mark.skipif(not ref_shims.available(), reason="no staged reference under oracle/_ref")


@needs_ref
def test_oracle_equals_staged_reference_prefill_and_decode():
    ns = ref_shims.reference(model=False)
    torch.manual_seed(3)
    B, H, L, d, dv, steps = 2, 3, 45, 16, 32, 3
    m = ns.LinearAttention(d_model=H * dv, feature_map=ns.TaylorExp(input_dim=d), feature_dim=d, num_heads=H,
                           head_dim=dv).double()
    m.out_proj = torch.nn.Identity()
    q = torch.randn(B, H, L + steps, d, dtype=torch.float64) / 2
    k = torch.randn(B, H, L + steps, d, dtype=torch.float64) / 2
    v = torch.randn(B, H, L + steps, dv, dtype=torch.float64)
    m.is_inference = True
    with torch.no_grad():
        y, kv, ks = m.parallel_forward(torch.zeros(B, L, H * dv, dtype=torch.float64), q[:, :, :L], k[:, :, :L],
                                       v[:, :, :L])
    y_o, kv_o, ks_o = O.linattn_parallel(q[:, :, :L], k[:, :, :L], v[:, :, :L])
    assert rel_err(y_o.transpose(1, 2).reshape(B, L, H * dv), y) < 1e-12
    assert rel_err(kv_o, kv) < 1e-12 and rel_err(ks_o, ks) < 1e-12
    y_c, kv_c, ks_c = O.linattn_chunked(q[:, :, :L], k[:, :, :L], v[:, :, :L], chunk=16)
    assert rel_err(y_c, y_o) < 1e-12 and rel_err(kv_c, kv) < 1e-12
    kv, ks = kv.clone(), ks.clone()
    for s in range(steps):
        sl = slice(L + s, L + s + 1)
        with torch.no_grad():
            y_r = m.recurrent_forward(torch.zeros(B, 1, H * dv, dtype=torch.float64), kv, ks,
                                      m.feature_map(q[:, :, sl]), m.feature_map(k[:, :, sl]), v[:, :, sl])
        y_s = O.linattn_recurrent_step(kv_o, ks_o, q[:, :, sl], k[:, :, sl], v[:, :, sl])
        assert rel_err(y_s.transpose(1, 2).reshape(B, 1, H * dv), y_r) < 1e-12
        assert rel_err(kv_o, kv) < 1e-12 and rel_err(ks_o, ks) < 1e-12


@needs_ref
def test_reference_factory_builds_b200_mixers_with_sliding_window_additions():
    from based_b200 import mixers
    ns = ref_shims.reference()
    cfg = ref_shims.based_config(ns, n_embd=128, n_layer=4, n_head=2, n_inner=256, vocab_size=97, alt_mixer_layers=[1],
                                 alt_mixer_2_layers=[2], l_max=64, window_size=128, targets="b200")
    assert "slide" in cfg.alt_mixer_2["_target_"]
    model = ns.GPTLMHeadModel(cfg)
    kinds = [type(layer.mixer) for layer in model.transformer.layers]
    assert kinds == [mixers.BaseConv, mixers.LinearAttention, mixers.SlidingAttention, mixers.BaseConv]
    slide = model.transformer.layers[2].mixer
    # what sliding_window_additions (gpt.py:99-145) injects: whole-head rotary, no biases, 1/sqrt(head_dim)
    assert slide.rotary_emb_dim == 64 and slide.window == (64, 0) and slide.layer_idx == 2
    assert slide.Wqkv.bias is None and slide.out_proj.bias is None
    assert slide.softmax_scale == pytest.approx(64 ** -0.5)
    reference_keys = ns.GPTLMHeadModel(ref_shims.based_config(
        ns, n_embd=128, n_layer=4, n_head=2, n_inner=256, vocab_size=97, alt_mixer_layers=[1], alt_mixer_2_layers=[2],
        l_max=64, window_size=128, targets="reference")).state_dict().keys()
    assert list(model.state_dict().keys()) == list(reference_keys)


def test_integration_notes_name_a_sliding_window_target_containing_slide():
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    targets = re.findall(r"_target_:\s*(based_b200[\w.]*)", text)
    assert targets, "INTEGRATION.md lists no based_b200 _target_ paths"
    import importlib
    for t in targets:
        mod, _, attr = t.rpartition(".")
        cls = getattr(importlib.import_module(mod), attr)          # every path resolves
        if cls.__name__ == "SlidingAttention":
            assert "slide" in t, f"{t}: gpt.py:87 applies sliding_window_additions only to paths containing 'slide'"
