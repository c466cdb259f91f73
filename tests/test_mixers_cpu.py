"""Host-side behaviour of the drop-in mixers that needs no GPU: parameter names and shapes
(checkpoint compatibility with the reference), cache shapes, argument checks."""
import pytest
import torch

from based_b200.generation import InferenceParams
from based_b200.mixers import LinearAttention, SlidingAttention, TaylorExp


def test_linear_attention_parameters_match_reference_layout():
    m = LinearAttention(d_model=1024, feature_map=TaylorExp(input_dim=16), feature_dim=16, num_heads=16,
                        head_dim=64, layer_idx=3)
    shapes = {k: tuple(v.shape) for k, v in m.state_dict().items()}
    # based/models/mixers/linear_attention.py:106-109
    assert shapes == {"proj_q.weight": (256, 1024), "proj_k.weight": (256, 1024),
                      "proj_v.weight": (1024, 1024), "out_proj.weight": (1024, 1024)}
    assert m.expanded_size() == 273
    kv, ks = m.allocate_inference_cache(4, 2048, dtype=torch.float32)
    assert kv.shape == (4, 16, 1, 64, 273) and ks.shape == (4, 16, 1, 1, 273)  # :261-266
    assert kv.abs().max() == 0 and ks.abs().max() == 0


def test_linear_attention_default_head_dim_and_1b_shape():
    m = LinearAttention(d_model=1792, feature_map=TaylorExp(input_dim=16), num_heads=16)
    assert m.head_dim == 112  # d_model // num_heads (:101)
    kv, _ = m.allocate_inference_cache(1, 16)
    assert kv.shape == (1, 16, 1, 112, 273)


def test_linear_attention_rejects_unknown_implementation():
    with pytest.raises(ValueError):
        LinearAttention(64, feature_map=TaylorExp(16), num_heads=2, parallel_implementation="tk")
    with pytest.raises(ValueError):
        LinearAttention(64, feature_map=TaylorExp(16), num_heads=2, feature_dim=8)


def test_taylor_exp_matches_golden():
    from conftest import load_golden, rel_err
    g = load_golden("taylor_exp.npz")
    assert rel_err(TaylorExp(16)(g["x"]), g["phi"]) < 1e-14


def test_mixers_have_no_cpu_path():
    m = LinearAttention(64, feature_map=TaylorExp(16), num_heads=2, head_dim=32)
    with pytest.raises(RuntimeError):
        m(torch.zeros(1, 4, 64))


def test_sliding_attention_parameters_and_cache():
    s = SlidingAttention(1024, 16, qkv_proj_bias=False, out_proj_bias=False, rotary_emb_dim=64, window_size=128,
                         layer_idx=2)
    shapes = {k: tuple(v.shape) for k, v in s.state_dict().items()}
    assert shapes == {"Wqkv.weight": (3072, 1024), "out_proj.weight": (1024, 1024)}  # slide_attention.py:365,:372
    assert s.window == (64, 0)  # :336: the argument is halved; 64 previous keys + self
    cache = s.allocate_inference_cache(3, 100, dtype=torch.bfloat16)
    assert cache.shape == (3, 100, 2, 16, 64)  # :374-377
    with pytest.raises(NotImplementedError):
        SlidingAttention(1024, 16, num_heads_kv=4)


def test_inference_params_mirror():
    ip = InferenceParams(max_seqlen=10, max_batch_size=2)
    ip.seqlen_offset = 5
    ip.reset(20, 4)
    assert (ip.max_seqlen, ip.max_batch_size, ip.seqlen_offset) == (20, 4, 0)
    assert ip.key_value_memory_dict == {}


def test_baseconv_mirror_keeps_the_reference_interface():
    """Parameter names / shapes and cache layout of based/models/mixers/convolution.py:174-217; no CPU path."""
    import pytest
    import torch
    from based_b200.mixers import BaseConv
    m = BaseConv(d_model=64, l_max=128, kernel_size=3, layer_idx=4)
    sd = {k: tuple(v.shape) for k, v in m.state_dict().items()}
    assert sd == {"in_proj.weight": (128, 64), "in_proj.bias": (128,), "out_proj.weight": (64, 64),
                  "out_proj.bias": (64,), "conv.conv.weight": (64, 1, 3)}
    cache = m.allocate_inference_cache(batch_size=3, max_seqlen=128)
    assert set(cache) == {"conv"} and cache["conv"].shape == (3, 64, 3)
    assert m.conv.layer_idx == (4, "conv")
    with pytest.raises(RuntimeError):  # CPU tensors are refused, there is no fallback
        m(torch.randn(1, 5, 64))


def test_model_assembly_keeps_the_reference_parameter_names():
    """Module tree of based/models/gpt.py:737-830 / block.py:27-93 (checked against the reference's own
    state dict in tests/golden/full_model.npz) and the per-layer cache layout."""
    import torch
    from conftest import load_golden
    from based_b200.model import BasedConfig, BasedLMHeadModel
    g = load_golden("full_model.npz")
    ref = {k[3:]: tuple(v.shape) for k, v in g.items() if k.startswith("sd.")}
    cfg = BasedConfig(n_embd=32, n_layer=3, n_head=2, n_inner=64, vocab_size=97, alt_mixer_layers=[1],
                      alt_mixer_2_layers=[], l_max=64)
    m = BasedLMHeadModel(cfg)
    mine = {k: tuple(v.shape) for k, v in m.state_dict().items() if k != "lm_head.weight"}
    assert mine == ref
    assert m.lm_head.weight is m.transformer.embeddings.word_embeddings.weight
    cache = m.allocate_inference_cache(2, 32, dtype=torch.float32)
    assert set(cache) == {0, 1, 2} and set(cache[0]) == {"conv"} and len(cache[1]) == 2
    full = BasedConfig.based_360m()
    assert full.padded_vocab_size == 50280 and len(full.alt_mixer_layers) == 5


def test_sample_token_policy():
    """Greedy, top-k support, nucleus support and temperature of the sampling policy (host logic, CPU tensors)."""
    import torch
    from based_b200.model import sample_token
    torch.manual_seed(0)
    logits = torch.tensor([[2.0, 1.0, 0.5, -1.0, -3.0], [0.0, 3.0, 2.9, -2.0, 1.0]])
    assert sample_token(logits).tolist() == [0, 1]
    many = logits.repeat_interleave(400, dim=0)
    topk = sample_token(many, top_k=2)
    assert set(topk[:400].tolist()) == {0, 1} and set(topk[400:].tolist()) == {1, 2}
    # nucleus: row 0 probabilities ~ [0.61, 0.22, 0.14, 0.03, 0.004]; top_p = 0.8 keeps the smallest head whose
    # mass reaches 0.8 -> tokens 0 and 1; row 1 ~ [0.024, 0.48, 0.43, 0.003, 0.065] -> tokens 1 and 2
    nuc = sample_token(many, top_k=0, top_p=0.8)
    assert set(nuc[:400].tolist()) == {0, 1} and set(nuc[400:].tolist()) == {1, 2}
    # a very low temperature makes sampling greedy; top_p outside (0, 1) filters nothing
    assert sample_token(many, top_k=5, temperature=1e-3).tolist() == [0] * 400 + [1] * 400
    assert len(set(sample_token(many, top_k=0, top_p=0.0, temperature=3.0)[:400].tolist())) >= 4
