"""Generate golden vectors for the sliding-window path from flash-attn on a CUDA device.

The reference's SlidingAttention has no CPU implementation: its arithmetic is flash-attn
(call sites based/models/mixers/slide_attention.py:100-106, :206-213, :414-427).  This
script calls the same flash-attn functions with the same arguments the reference passes
(causal=True, window_size=(window_left, 0), rotary tables, cache_seqlens) on seeded inputs
and stores inputs and outputs.  Usage (GPU required)::

    python tests/golden/make_swa_golden_gpu.py <output.npz>

Copy the output to tests/golden/swa_flash.npz.  The tests only read that file.
"""
import sys

import numpy as np
import torch


def main(out_path):
    from flash_attn import flash_attn_qkvpacked_func, flash_attn_with_kvcache
    import flash_attn

    torch.manual_seed(0)
    dev = "cuda"
    out = {"flash_attn_version": np.array(flash_attn.__version__)}
    # prefill: packed qkv [B, L, 3, H, hd], window 64
    for name, (B, L, H, hd, w) in {"p64": (2, 200, 3, 64, 64), "p112": (1, 150, 2, 112, 64),
                                   "p64w128": (1, 300, 2, 64, 128)}.items():
        qkv = torch.randn(B, L, 3, H, hd, device=dev).bfloat16()
        o = flash_attn_qkvpacked_func(qkv, 0.0, softmax_scale=hd ** -0.5, causal=True, window_size=(w, 0))
        out[f"{name}_qkv"] = qkv.float().cpu().numpy()
        out[f"{name}_out"] = o.float().cpu().numpy()
        out[f"{name}_w"] = np.array(w)
    # decode with rotary + cache append (slide_attention.py:414-427)
    B, H, hd, maxL, w = 2, 3, 64, 120, 64
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))
    freqs = torch.outer(torch.arange(maxL, dtype=torch.float32), inv_freq)
    cos, sin = torch.cos(freqs).bfloat16().to(dev), torch.sin(freqs).bfloat16().to(dev)
    cache = torch.randn(B, maxL, 2, H, hd, device=dev).bfloat16()
    out["d_cache_in"] = cache.float().cpu().numpy()
    lens = torch.tensor([70, 100], dtype=torch.int32, device=dev)
    outs, qs, ks, vs = [], [], [], []
    for step in range(3):
        q = torch.randn(B, 1, H, hd, device=dev).bfloat16()
        k = torch.randn(B, 1, H, hd, device=dev).bfloat16()
        v = torch.randn(B, 1, H, hd, device=dev).bfloat16()
        o = flash_attn_with_kvcache(q, cache[:, :, 0], cache[:, :, 1], k, v, rotary_cos=cos, rotary_sin=sin,
                                    cache_seqlens=lens, softmax_scale=hd ** -0.5, causal=True,
                                    rotary_interleaved=False, window_size=(w, 0))
        outs.append(o.float().cpu()); qs.append(q.float().cpu()); ks.append(k.float().cpu()); vs.append(v.float().cpu())
        lens = lens + 1
    out["d_q"] = torch.stack(qs).numpy(); out["d_k"] = torch.stack(ks).numpy(); out["d_v"] = torch.stack(vs).numpy()
    out["d_out"] = torch.stack(outs).numpy()
    out["d_cache_out"] = cache.float().cpu().numpy()
    out["d_lens0"] = np.array([70, 100]); out["d_w"] = np.array(w)
    np.savez_compressed(out_path, **out)
    print("wrote", out_path)


if __name__ == "__main__":
    main(sys.argv[1])
