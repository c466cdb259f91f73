"""Inference-only assembly of the Based language model on the B200 kernels.

Mirrors the module tree and parameter names of the reference's ``GPTLMHeadModel``
(based/models/gpt.py:737-830: ``transformer.embeddings.word_embeddings``, ``transformer.layers.N``
with ``mixer`` / ``norm1`` / ``mlp`` / ``norm2`` as in based/models/block.py:27-93,
``transformer.ln_f``, ``lm_head`` tied to the embedding, gpt.py:781-785), so a reference
checkpoint loads with ``load_state_dict``.  Only what generation needs is here: the prenorm
block of block.py:134-163 with an fp32 residual stream, layer selection by index as
``create_mixer_cls`` does it (gpt.py:64-96), greedy decoding with the prompt pass / single-token
steps split of based/generation.py:93-204, and optional CUDA-graph replay of the decode step
(:689-739).  Training, dropout, tensor-parallel embeddings and sampling strategies are not.
"""
from dataclasses import dataclass, field
from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .generation import InferenceParams
from .mixers import BaseConv, LinearAttention, SlidingAttention, TaylorExp
from .modules import GatedMlp, RMSNorm


def sample_token(logits: torch.Tensor, top_k: int = 1, top_p: float = 0.0, temperature: float = 1.0) -> torch.Tensor:
    """Next token per row of ``logits [B, V]``: greedy for ``top_k == 1``; otherwise restrict to the ``top_k`` largest
    logits (all of them for ``top_k <= 0``), divide by ``temperature``, drop the low-probability tail whose
    cumulative probability is at most ``1 - top_p`` (nucleus sampling; no-op for ``top_p`` outside (0, 1)), and draw
    from the softmax of what is left.  Same policy as ``sample`` in based/generation.py:38-92."""
    if top_k == 1:
        return logits.argmax(dim=-1)
    if not 0.0 <= top_p <= 1.0:
        raise ValueError("top_p must be in [0, 1]")
    if top_k > 0:
        vals, idx = torch.topk(logits, min(top_k, logits.size(-1)), dim=-1)       # descending
    else:
        vals, idx = torch.sort(logits, dim=-1, descending=True)
    vals = vals.float()
    if temperature != 1.0:
        vals = vals / temperature
    if 0.0 < top_p < 1.0:
        probs = vals.softmax(dim=-1)
        tail = probs.flip(-1).cumsum(dim=-1).flip(-1)     # mass of this candidate and everything less likely
        vals = vals.masked_fill(tail <= 1.0 - top_p, float("-inf"))
    choice = torch.multinomial(vals.softmax(dim=-1), num_samples=1)
    return idx.gather(-1, choice).squeeze(-1)


@dataclass
class BasedConfig:
    """The fields of the reference's experiment configs that shape the model
    (train/configs/experiment/reference/based-360m.yaml:49-117)."""
    n_embd: int = 1024
    n_layer: int = 27
    n_head: int = 16
    n_inner: Optional[int] = None              # GatedMlp hidden size; None -> 2 * n_embd as in the configs
    vocab_size: int = 50277
    pad_vocab_size_multiple: int = 8
    layer_norm_epsilon: float = 1e-5
    alt_mixer_layers: List[int] = field(default_factory=lambda: [1, 6, 11, 16, 21])      # LinearAttention
    alt_mixer_2_layers: List[int] = field(default_factory=lambda: [2, 7, 12, 17, 22])    # SlidingAttention
    conv_expand_proj: int = 4
    conv_kernel_size: int = 3
    feature_dim: int = 16
    window_size: int = 128                     # SlidingAttention window_size; the kernel window is window_size // 2
    rotary_emb_fraction: float = 1.0
    residual_in_fp32: bool = True
    l_max: int = 2048

    @property
    def padded_vocab_size(self):
        m = self.pad_vocab_size_multiple
        return (self.vocab_size + m - 1) // m * m

    @classmethod
    def based_360m(cls):
        return cls()

    @classmethod
    def based_1b(cls):
        """train/configs/experiment/reference/based-1b.yaml:50-123."""
        return cls(n_embd=1792, n_layer=36, alt_mixer_layers=[1, 6, 11, 16, 21, 27, 33],
                   alt_mixer_2_layers=[2, 7, 12, 17, 22, 28, 34])


class Block(nn.Module):
    """Prenorm block: add -> norm -> mixer -> add -> norm -> MLP, returning (hidden, residual)."""

    def __init__(self, config: BasedConfig, layer_idx: int, device=None, dtype=None):
        super().__init__()
        fk = {"device": device, "dtype": dtype}
        d = config.n_embd
        self.layer_idx = layer_idx
        self.residual_in_fp32 = config.residual_in_fp32
        if layer_idx in config.alt_mixer_layers:
            self.mixer = LinearAttention(d, feature_map=TaylorExp(input_dim=config.feature_dim), l_max=config.l_max,
                                         feature_dim=config.feature_dim, num_heads=config.n_head, layer_idx=layer_idx,
                                         fuse_qkv=True, **fk)
        elif layer_idx in config.alt_mixer_2_layers:
            head_dim = d // config.n_head
            self.mixer = SlidingAttention(d, num_heads=config.n_head, window_size=config.window_size, causal=True,
                                          qkv_proj_bias=False, out_proj_bias=False, layer_idx=layer_idx,
                                          rotary_emb_dim=int(config.rotary_emb_fraction * head_dim), **fk)
        else:
            self.mixer = BaseConv(d, l_max=config.l_max, kernel_size=config.conv_kernel_size, layer_idx=layer_idx,
                                  use_bias=True, expand_proj=config.conv_expand_proj, **fk)
        self.norm1 = RMSNorm(d, eps=config.layer_norm_epsilon, **fk)
        self.mlp = GatedMlp(d, hidden_features=config.n_inner or 2 * d, activation=F.silu, bias1=False, bias2=False, **fk)
        self.norm2 = RMSNorm(d, eps=config.layer_norm_epsilon, **fk)

    def allocate_inference_cache(self, batch_size, max_seqlen, dtype=None, **kwargs):
        return self.mixer.allocate_inference_cache(batch_size, max_seqlen, dtype=dtype, **kwargs)

    def forward(self, hidden_states, residual=None, inference_params=None):
        # block.py:134-137: residual = hidden + residual; hidden = norm(residual.to(weight dtype)); residual kept in fp32
        hidden_states, residual = self.norm1(hidden_states, residual=residual, prenorm=True,
                                             residual_in_fp32=self.residual_in_fp32, round_input=True)
        hidden_states = self.mixer(hidden_states, inference_params=inference_params)
        hidden_states, residual = self.norm2(hidden_states, residual=residual, prenorm=True,
                                             residual_in_fp32=self.residual_in_fp32, round_input=True)
        return self.mlp(hidden_states), residual


class _Embeddings(nn.Module):
    def __init__(self, embed_dim, vocab_size, device=None, dtype=None):
        super().__init__()
        self.word_embeddings = nn.Embedding(vocab_size, embed_dim, device=device, dtype=dtype)

    def forward(self, input_ids):
        return self.word_embeddings(input_ids)


class BasedModel(nn.Module):
    def __init__(self, config: BasedConfig, device=None, dtype=None):
        super().__init__()
        self.config = config
        self.embeddings = _Embeddings(config.n_embd, config.padded_vocab_size, device=device, dtype=dtype)
        self.layers = nn.ModuleList([Block(config, i, device=device, dtype=dtype) for i in range(config.n_layer)])
        self.ln_f = RMSNorm(config.n_embd, eps=config.layer_norm_epsilon, device=device, dtype=dtype)

    def allocate_inference_cache(self, batch_size, max_seqlen, dtype=None, **kwargs):
        return {i: layer.allocate_inference_cache(batch_size, max_seqlen, dtype=dtype, **kwargs)
                for i, layer in enumerate(self.layers)}

    def forward(self, input_ids, inference_params=None):
        hidden_states, residual = self.embeddings(input_ids), None
        for layer in self.layers:
            hidden_states, residual = layer(hidden_states, residual, inference_params=inference_params)
        # gpt.py:676-690: last add, then the final norm on the sum cast to the weights' dtype
        return self.ln_f(hidden_states, residual=residual, residual_in_fp32=self.config.residual_in_fp32,
                         round_input=True)


class BasedLMHeadModel(nn.Module):
    def __init__(self, config: BasedConfig, device=None, dtype=None):
        super().__init__()
        self.config = config
        self.transformer = BasedModel(config, device=device, dtype=dtype)
        self.lm_head = nn.Linear(config.n_embd, config.padded_vocab_size, bias=False, device=device, dtype=dtype)
        self.tie_weights()

    def tie_weights(self):
        self.lm_head.weight = self.transformer.embeddings.word_embeddings.weight

    def allocate_inference_cache(self, batch_size, max_seqlen, dtype=None, **kwargs):
        return self.transformer.allocate_inference_cache(batch_size, max_seqlen, dtype=dtype, **kwargs)

    def forward(self, input_ids, inference_params=None, num_last_tokens=0):
        """Logits ``[B, L, padded_vocab]`` (the last ``num_last_tokens`` positions when > 0), gpt.py:794-830."""
        hidden_states = self.transformer(input_ids, inference_params=inference_params)
        if num_last_tokens > 0:
            hidden_states = hidden_states[:, -num_last_tokens:]
        return ops.linear(hidden_states, self.lm_head.weight, self.lm_head.bias)

    @torch.inference_mode()
    def generate(self, input_ids, max_new_tokens: int, cg: bool = False, timings: Optional[dict] = None,
                 top_k: int = 1, top_p: float = 0.0, temperature: float = 1.0):
        """Decoding: one prompt pass, then one token per step (generation.py:93-204); greedy by default, top-k /
        nucleus / temperature sampling as :func:`sample_token` otherwise.  With ``cg`` the decode step is
        captured once in a CUDA graph and replayed (:689-739).  Returns ``[B, L + max_new_tokens]``.
        ``timings``, when given, receives device times in ms: ``prefill_ms``, ``decode_ms`` (all steps)."""
        B, L = input_ids.shape
        dtype = self.lm_head.weight.dtype
        ip = InferenceParams(max_seqlen=L + max_new_tokens, max_batch_size=B)
        ip.key_value_memory_dict = self.allocate_inference_cache(B, ip.max_seqlen, dtype=dtype)
        ip.lengths_per_sample = torch.full((B,), L, dtype=torch.int32, device=input_ids.device)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        out = torch.empty(B, L + max_new_tokens, dtype=input_ids.dtype, device=input_ids.device)
        out[:, :L] = input_ids
        ev[0].record()
        logits = self.forward(input_ids, inference_params=ip, num_last_tokens=1)
        token = sample_token(logits[:, -1, : self.config.vocab_size], top_k, top_p, temperature).unsqueeze(-1)
        ev[1].record()
        ip.seqlen_offset = L
        if max_new_tokens > 0:
            out[:, L] = token[:, 0]
        cur = token.clone()

        def step():
            lg = self.forward(cur, inference_params=ip, num_last_tokens=1)
            cur.copy_(sample_token(lg[:, -1, : self.config.vocab_size], top_k, top_p, temperature).unsqueeze(-1))
            ip.lengths_per_sample.add_(1)

        graph = None
        steps_left = max_new_tokens - 1
        if cg and steps_left > 2:
            # warm-up on a side stream (the first calls may build rotary tables), then capture one step
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            saved = self._snapshot_state(ip, cur)
            with torch.cuda.stream(s):
                for _ in range(2):
                    step()
            torch.cuda.current_stream().wait_stream(s)
            self._restore_state(ip, cur, saved)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            self._restore_state(ip, cur, saved)
        for i in range(steps_left):
            if graph is not None:
                graph.replay()
            else:
                step()
            ip.seqlen_offset += 1
            out[:, L + 1 + i] = cur[:, 0]
        ev[2].record()
        if timings is not None:
            torch.cuda.synchronize()
            ops.check_status()   # the device is idle here: a tensor-core kernel that gave up on a wait shows now
            timings["prefill_ms"] = ev[0].elapsed_time(ev[1])
            timings["decode_ms"] = ev[1].elapsed_time(ev[2])
        return out

    @staticmethod
    def _flat_state(ip):
        for v in ip.key_value_memory_dict.values():
            if isinstance(v, dict):
                yield from v.values()
            elif isinstance(v, (tuple, list)):
                yield from v
            else:
                yield v

    def _snapshot_state(self, ip, cur):
        return [t.clone() for t in self._flat_state(ip)] + [ip.lengths_per_sample.clone(), cur.clone()]

    def _restore_state(self, ip, cur, saved):
        tensors = list(self._flat_state(ip)) + [ip.lengths_per_sample, cur]
        for t, s in zip(tensors, saved):
            t.copy_(s)
