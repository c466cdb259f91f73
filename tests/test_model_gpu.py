"""The inference-only model assembly on the GPU kernels against the reference's GPTLMHeadModel
(golden logits) and against itself (step-by-step decoding == a longer prompt pass; CUDA-graph
replay == eager).  Tolerances on logits: relative error 1e-3 in fp32 (the GEMMs are cuBLAS fp32),
5e-2 in bf16."""
import pytest
import torch

from conftest import load_golden, rel_err

pytestmark = pytest.mark.gpu


def _golden_model(dtype):
    from based_b200.model import BasedConfig, BasedLMHeadModel
    g = load_golden("full_model.npz")
    cfg = BasedConfig(n_embd=32, n_layer=3, n_head=2, n_inner=64, vocab_size=97, alt_mixer_layers=[1],
                      alt_mixer_2_layers=[], l_max=64)
    m = BasedLMHeadModel(cfg)
    sd = {k[3:]: torch.as_tensor(v) for k, v in g.items() if k.startswith("sd.")}
    missing, unexpected = m.load_state_dict(sd, strict=False)
    assert unexpected == [] and missing == ["lm_head.weight"]      # tied to the embedding
    m.tie_weights()
    return m.to(device="cuda", dtype=dtype).eval(), g


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_model_matches_reference_logits(dtype):
    from based_b200.generation import InferenceParams
    m, g = _golden_model(dtype)
    tol = 1e-3 if dtype == torch.float32 else 5e-2
    ids = torch.as_tensor(g["input_ids"]).cuda()
    with torch.inference_mode():
        assert rel_err(m(ids).float().cpu(), torch.as_tensor(g["logits_full"])) < tol
        ip = InferenceParams(max_seqlen=32, max_batch_size=2)
        last = m(ids, inference_params=ip, num_last_tokens=1)
        assert rel_err(last.float().cpu(), torch.as_tensor(g["logits_prefill_last"])) < tol
        for i in range(3):
            ip.seqlen_offset = ids.shape[1] + i
            lg = m(torch.as_tensor(g[f"step{i}_ids"]).cuda(), inference_params=ip, num_last_tokens=1)
            assert rel_err(lg.float().cpu(), torch.as_tensor(g[f"step{i}_logits"])) < tol


def _small_model(dtype=torch.bfloat16, seed=0):
    from based_b200.model import BasedConfig, BasedLMHeadModel
    torch.manual_seed(seed)
    cfg = BasedConfig(n_embd=128, n_layer=4, n_head=2, n_inner=256, vocab_size=211, alt_mixer_layers=[1],
                      alt_mixer_2_layers=[2], window_size=32, l_max=256)
    m = BasedLMHeadModel(cfg, device="cuda", dtype=dtype).eval()
    with torch.no_grad():
        for name, p in m.named_parameters():
            if p.dim() > 1:
                p.normal_(0, 0.08)
    return m


def test_decode_steps_equal_a_longer_prompt_pass():
    """All three mixer kinds (conv, linear attention, sliding window with rotary): prompt pass + n single-token
    steps give the logits of one pass over the longer sequence (the reference's generation test property,
    based/tests/test_generation.py:106-115, bf16 tolerances)."""
    from based_b200.generation import InferenceParams
    m = _small_model()
    B, L, n = 3, 70, 6
    ids = torch.randint(0, 211, (B, L + n), device="cuda")
    with torch.inference_mode():
        full = m(ids).float()
        ip = InferenceParams(max_seqlen=L + n, max_batch_size=B)
        ip.key_value_memory_dict = m.allocate_inference_cache(B, L + n, dtype=torch.bfloat16)
        lg = m(ids[:, :L], inference_params=ip, num_last_tokens=1).float()
        assert torch.allclose(lg[:, 0], full[:, L - 1], atol=5e-2, rtol=1e-2)
        for i in range(n):
            ip.seqlen_offset = L + i
            lg = m(ids[:, L + i:L + i + 1], inference_params=ip, num_last_tokens=1).float()
            assert torch.allclose(lg[:, 0], full[:, L + i], atol=5e-2, rtol=1e-2), i


def test_generate_cuda_graph_equals_eager():
    m = _small_model(seed=1)
    ids = torch.randint(0, 211, (2, 40), device="cuda")
    t = {}
    eager = m.generate(ids, max_new_tokens=12, cg=False, timings=t)
    graphed = m.generate(ids, max_new_tokens=12, cg=True)
    assert eager.shape == (2, 52) and torch.equal(eager[:, :40], ids)
    assert torch.equal(eager, graphed)
    assert t["prefill_ms"] > 0 and t["decode_ms"] > 0
    # greedy continuation: the first generated token is the argmax of the prompt pass
    with torch.inference_mode():
        first = m(ids)[:, -1, :211].argmax(-1)
    assert torch.equal(eager[:, 40], first)


def test_generate_with_sampling():
    """Sampling decode: reproducible under a seed, tokens inside the vocabulary, and equal to greedy when the
    temperature is tiny; the CUDA-graph path accepts it too."""
    m = _small_model(seed=3)
    ids = torch.randint(0, 211, (3, 20), device="cuda")
    greedy = m.generate(ids, max_new_tokens=8)
    torch.manual_seed(5)
    a = m.generate(ids, max_new_tokens=8, top_k=20, top_p=0.9, temperature=0.8)
    torch.manual_seed(5)
    b = m.generate(ids, max_new_tokens=8, top_k=20, top_p=0.9, temperature=0.8)
    assert torch.equal(a, b) and int(a.max()) < 211 and int(a.min()) >= 0
    assert torch.equal(m.generate(ids, max_new_tokens=8, top_k=20, temperature=1e-4), greedy)
    g = m.generate(ids, max_new_tokens=8, cg=True, top_k=20, top_p=0.9, temperature=0.8)
    assert g.shape == (3, 28) and int(g.max()) < 211 and torch.equal(g[:, :20], ids)
