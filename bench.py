"""Benchmark of the Based hot path on B200.

Headline (the JSON line's ``value``): decode tok/s of the recurrent linear-attention step on
the decode microbench workload — bf16 q/k/v, fp32 state [B=256, H=16, 1, 64, 273], one token
per sequence per step.  One "step" is one pass of the decode kernel over the whole batch.
Per-GPU work is fixed as GPUs are added (batch x heads shards, no collective): weak scaling.

The same line carries: ``roofline`` (HBM fraction of the decode kernel), ``e2e`` (the same
step through the public API with host buffers: H2D of q/k/v and D2H of y inside the timed
region), ``cpu_baseline`` (the CPU oracle's restatement of the reference's recurrent_forward
on the host cores), ``prefill`` / ``swa`` (the prefill sweep: tok/s and roofline fractions),
``clocks`` sampled during the timed region.

``--impl reference`` times the CPU restatement of the reference's PyTorch code for the same
step on the host cores (the reference is pure Python/PyTorch for this path and cannot travel
to the GPU box; the oracle is pinned against it by golden vectors).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

B_DEC, H, D_FEAT, DV, D_EXP = 256, 16, 16, 64, 273
# algorithmic bytes per (batch, head) per decode step: state R+W, k_state R+W, q/k/v/y
DEC_BYTES_PER_UNIT = 2 * DV * D_EXP * 4 + 2 * D_EXP * 4 + 2 * (16 + 16 + DV + DV)
PREFILL_FLOP_PER_TOKEN_HEAD = 4 * D_EXP * (DV + 1)
PREFILL_BYTES_PER_TOKEN_HEAD = 2 * (16 + 16 + DV + DV)
SWA_BYTES_PER_TOKEN_HEAD = 4 * 64 * 2
SWA_FLOP_PER_TOKEN_HEAD = 4 * 65 * 64


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks/throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        self.t.join(timeout=2)
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            f = [x.strip() for x in s.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0])); mx = float(f[1])
            except ValueError:
                continue
            for n, val in zip(names, f[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def decode_inputs(B, pool, device, seed):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(pool, B, H, 16, generator=g) / 4).bfloat16()
    k = (torch.randn(pool, B, H, 16, generator=g) / 4).bfloat16()
    v = torch.randn(pool, B, H, DV, generator=g).bfloat16()
    kv = 0.02 * torch.randn(B, H, 1, DV, D_EXP, generator=g)
    ks = 0.02 * torch.randn(B, H, 1, 1, D_EXP, generator=g)
    return q, k, v, kv, ks


def cpu_decode_baseline(B, steps, warmup, seed=0):
    """The oracle's recurrent step (restating linear_attention.py:139, :230-251) on the host cores."""
    from oracle import based_oracle as O
    q, k, v, kv, ks = decode_inputs(B, 4, "cpu", seed)
    q, k, v = q.unsqueeze(3), k.unsqueeze(3), v.unsqueeze(3)   # [pool, B, H, 1, .]
    for i in range(warmup):
        O.linattn_recurrent_step(kv, ks, q[i % 4], k[i % 4], v[i % 4])
    t0 = time.perf_counter()
    for i in range(steps):
        O.linattn_recurrent_step(kv, ks, q[i % 4], k[i % 4], v[i % 4])
    dt = time.perf_counter() - t0
    return B * steps / dt, dt


def use_all_host_threads():
    """torchrun exports OMP_NUM_THREADS=1; the CPU legs are meant to use every host core."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(max(1, n))
    return n


def run_reference(args, rank, world):
    if rank != 0:
        return
    use_all_host_threads()
    Bs = 32
    tput, dt = cpu_decode_baseline(Bs, args.steps, args.warmup)
    cores = torch.get_num_threads()
    sample = (f"each step = one recurrent step on B={Bs} of the 256 sequences (H=16, fp32 state, bf16 q/k/v), "
              f"{args.steps} steps, CPU restatement of recurrent_forward")
    line = {
        "impl": "reference", "metric": "decode_tok_per_s", "value": tput, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "decode microbench: B=256,H=16,d=16,dv=64, fp32 state [B,H,1,64,273], bf16 q/k/v, "
                               "1 token/step"},
        "cpu_baseline": {"value": tput, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tput, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "host_cpus": os.cpu_count(),
    }
    print(json.dumps(line), flush=True)


def time_kernel(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters  # ms


def time_graph(fn, iters, replays=3):
    """Device time per call of a launch too short to time through Python: `iters` calls captured in
    one CUDA graph on a side stream, the graph replayed between two events."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(3):
            fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(iters):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (iters * replays)  # ms


def prefill_sweep(ops, peaks, lengths):
    """Prefill sweep: B=8, H=16, d=16, dv=64, bf16, q/k/v ~ N(0,1)/4; linear attention and window-64 SWA."""
    out_lin, out_swa = [], []
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    for L in lengths:
        g = torch.Generator(device="cuda").manual_seed(L)
        q = (torch.randn(8, H, L, 16, device="cuda", generator=g) / 4).bfloat16()
        k = (torch.randn(8, H, L, 16, device="cuda", generator=g) / 4).bfloat16()
        v = (torch.randn(8, H, L, DV, device="cuda", generator=g) / 4).bfloat16()
        y = torch.empty(8, L, H, DV, dtype=torch.bfloat16, device="cuda").permute(0, 2, 1, 3)
        kv = torch.empty(8, H, 1, DV, D_EXP, device="cuda")
        ks = torch.empty(8, H, 1, 1, D_EXP, device="cuda")

        def lin():
            flush.zero_()
            ops.linattn_prefill(q, k, v, out=y, kv_state=kv, k_state=ks)

        def fl():
            flush.zero_()

        iters = 5 if L >= 32768 else 10
        t = time_kernel(lin, iters) - time_kernel(fl, iters)
        units = 8 * H * L
        out_lin.append({"L": L, "ms": t, "tok_per_s": 8 * L / (t * 1e-3),
                        "tensor_frac": units * PREFILL_FLOP_PER_TOKEN_HEAD / (t * 1e-3) / (peaks["bf16_tflops"] * 1e12),
                        "hbm_frac": units * PREFILL_BYTES_PER_TOKEN_HEAD / (t * 1e-3) / (peaks["hbm_gbs"] * 1e9)})
        qkv = (torch.randn(8, L, 3, H, 64, device="cuda", generator=g) / 4).bfloat16()
        o = torch.empty(8, L, H, 64, dtype=torch.bfloat16, device="cuda")

        def swa():
            flush.zero_()
            ops.swa_prefill(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], 64, out=o)

        t = time_kernel(swa, iters) - time_kernel(fl, iters)
        out_swa.append({"L": L, "ms": t, "tok_per_s": 8 * L / (t * 1e-3),
                        "hbm_frac": units * SWA_BYTES_PER_TOKEN_HEAD / (t * 1e-3) / (peaks["hbm_gbs"] * 1e9),
                        "tensor_frac": units * SWA_FLOP_PER_TOKEN_HEAD / (t * 1e-3) / (peaks["bf16_tflops"] * 1e12)})
        del q, k, v, y, qkv, o
    return out_lin, out_swa


def gated_conv_bench(ops, peaks):
    """BaseConv's gated short convolution at the 360M model's layer size and the generation benchmark's
    prompt (B=16, L=2048, d_inner=1024, k=3, bf16): algorithmic bytes = 3 elements per (token, channel)."""
    B, L, di, k = 16, 2048, 1024, 3
    g = torch.Generator(device="cuda").manual_seed(3)
    u = torch.randn(B, L, 2 * di, device="cuda", generator=g).bfloat16()
    w = (torch.randn(di, k, device="cuda", generator=g) * 0.5).bfloat16()
    out = torch.empty(B, L, di, dtype=torch.bfloat16, device="cuda")
    state = torch.empty(B, di, k, dtype=torch.bfloat16, device="cuda")
    t = time_graph(lambda: ops.gated_conv_prefill(u, w, state=state, out=out), 20)
    nbytes = B * L * di * 3 * 2
    u_t, y_t = u[:, 0], out[:, 0]
    ts = time_graph(lambda: ops.gated_conv_step(u_t, state, w, out=y_t), 50)
    return {"B": B, "L": L, "d_inner": di, "k": k, "ms": t, "tok_per_s": B * L / (t * 1e-3),
            "hbm_frac": nbytes / (t * 1e-3) / (peaks["hbm_gbs"] * 1e9), "bytes": nbytes,
            "l2": "working set 201 MB > L2", "timing": "CUDA graph of 20 launches", "step_us": ts * 1e3}


def norm_act_bench(ops, peaks):
    """Residual add + RMSNorm (bf16 activations, fp32 residual stream in and out) and the SwiGLU activation at
    the 360M model's sizes: M = 16 x 2048 rows, D = 1024, F = 2816."""
    M, D, Fh = 16 * 2048, 1024, 2816
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(M, D, device="cuda", generator=g).bfloat16()
    res = torch.randn(M, D, device="cuda", generator=g)
    w = torch.ones(D, device="cuda").bfloat16()
    y = torch.randn(M, 2 * Fh, device="cuda", generator=g).bfloat16()
    from based_b200 import _capi
    lib = _capi.lib()
    out = torch.empty_like(x)
    res_out = torch.empty_like(res)
    h = torch.empty(M, Fh, dtype=torch.bfloat16, device="cuda")
    st = torch.cuda.current_stream

    def norm():
        _capi.check(lib.based_add_rmsnorm(x.data_ptr(), res.data_ptr(), w.data_ptr(), None, out.data_ptr(),
                                          res_out.data_ptr(), M, D, D, D, D, D, 1e-5, 1, 0, 1, 0, st().cuda_stream), "norm")

    def act():
        _capi.check(lib.based_gated_act(y.data_ptr(), y.data_ptr() + 2 * Fh, h.data_ptr(), M, Fh, 2 * Fh, 2 * Fh, Fh,
                                        0, 1, st().cuda_stream), "act")

    tn, ta = time_graph(norm, 20), time_graph(act, 20)
    bn, ba = M * D * 12, M * Fh * 6
    return {"rows": M, "D": D, "F": Fh, "timing": "CUDA graph of 20 launches",
            "add_rmsnorm": {"ms": tn, "bytes": bn, "hbm_frac": bn / (tn * 1e-3) / (peaks["hbm_gbs"] * 1e9)},
            "gated_act": {"ms": ta, "bytes": ba, "hbm_frac": ba / (ta * 1e-3) / (peaks["hbm_gbs"] * 1e9)}}


def generation_bench(B=16, L=2048, new_tokens=512, size="360m"):
    """The 360M-parameter Based model (27 blocks: 17 BaseConv, 5 LinearAttention, 5 SlidingAttention) or the
    1.4B one (36 blocks: 22 / 7 / 7, d_model 1792, head_dim 112); bf16, random-init weights, synthetic token
    ids: one prompt pass over [B, L], then greedy single-token steps replayed from a CUDA graph.  Device times
    by CUDA events inside generate()."""
    from based_b200.model import BasedConfig, BasedLMHeadModel
    torch.manual_seed(0)
    cfg = BasedConfig.based_360m() if size == "360m" else BasedConfig.based_1b()
    cfg.l_max = L + new_tokens
    model = BasedLMHeadModel(cfg, device="cuda", dtype=torch.bfloat16).eval()
    with torch.no_grad():
        for prm in model.parameters():
            if prm.dim() > 1:
                prm.normal_(0, 0.02)
    nparam = sum(p.numel() for p in model.parameters())
    ids = torch.randint(0, cfg.vocab_size, (B, L), device="cuda")
    model.generate(ids, max_new_tokens=8, cg=True)   # warm-up at full size: allocator, cuBLAS heuristics, rotary tables
    t = {}
    out = model.generate(ids, max_new_tokens=new_tokens, cg=True, timings=t)
    assert out.shape == (B, L + new_tokens)
    steps = new_tokens - 1  # the first new token comes from the prompt pass
    res = {"model": f"based-{size} (random init)", "params": nparam, "B": B, "prompt": L, "new_tokens": new_tokens,
           "prefill_ms": t["prefill_ms"], "prefill_tok_per_s": B * L / (t["prefill_ms"] * 1e-3),
           "decode_ms_per_step": t["decode_ms"] / steps, "decode_tok_per_s": B * steps / (t["decode_ms"] * 1e-3),
           "decode": f"CUDA graph replay of one step ({cfg.n_layer} blocks + lm_head + argmax)"}
    del model
    torch.cuda.empty_cache()
    return res


def small_batch_prefill(ops, L):
    """One sequence (B=1, H=16, dv=64): one CTA per head against the sequence split the library picks."""
    g = torch.Generator(device="cuda").manual_seed(L + 1)
    q = (torch.randn(1, H, L, 16, device="cuda", generator=g) / 4).bfloat16()
    k = (torch.randn(1, H, L, 16, device="cuda", generator=g) / 4).bfloat16()
    v = (torch.randn(1, H, L, DV, device="cuda", generator=g) / 4).bfloat16()
    from based_b200 import _capi
    nseg = _capi.lib().based_linattn_prefill_segments(1, H, L)
    t1 = time_kernel(lambda: ops.linattn_prefill(q, k, v, nseg=1), 10)
    ts = time_kernel(lambda: ops.linattn_prefill(q, k, v, nseg=nseg), 10)
    return {"B": 1, "H": H, "L": L, "ms_one_cta_per_head": t1, "segments": nseg, "ms_sequence_split": ts,
            "tok_per_s": L / (ts * 1e-3), "l2": "inputs (3 MB) stay in L2 between iterations"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--strong", action="store_true",
                    help="strong scaling: split the one B=256 batch across the GPUs instead of one batch per GPU")
    ap.add_argument("--no-sweep", action="store_true", help="skip the prefill / SWA sweep")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--quick", action="store_true", help="prefill sweep at L=2048 only")
    ap.add_argument("--sweep-L", type=int, nargs="*", default=None, help="sequence lengths of the prefill sweep")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch.distributed as dist
    from based_b200 import build_library, ops
    build_library()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()
    K, W, pool = args.steps, args.warmup, 16
    # weak scaling (default, what the N-GPU launches measure): every rank runs the whole B=256 batch of its own;
    # --strong: the one B=256 batch is split across the ranks (B / N sequences each)
    Bd = B_DEC // world if args.strong else B_DEC

    qh, kh, vh, kv0, ks0 = decode_inputs(Bd, pool, "cpu", seed=rank)
    q, k, v = qh.to(dev), kh.to(dev), vh.to(dev)
    kv, ks = kv0.to(dev), ks0.to(dev)
    y = torch.empty(Bd, 1, H * DV, dtype=torch.bfloat16, device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---------------- device-resident timed region ----------------
    for i in range(W):
        ops.linattn_decode(q[i % pool], k[i % pool], v[i % pool], kv, ks, out=y)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    barrier()
    if sampler:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(K):
        ops.linattn_decode(q[i % pool], k[i % pool], v[i % pool], kv, ks, out=y)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if sampler else None
    assert torch.isfinite(y.float()).all()

    # ---------------- end to end: host buffers, H2D + kernel + D2H per step ----------------
    # Every step copies its q/k/v from pinned host memory and returns y to pinned host memory through
    # the public op.  The copies run on their own streams, double-buffered, so that step i+1's inputs
    # travel while step i computes (what a serving loop does); the state stays on the device.
    qp, kp, vp = qh.pin_memory(), kh.pin_memory(), vh.pin_memory()
    yh = [torch.empty(Bd, 1, H * DV, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    qd = [torch.empty_like(q[0]) for _ in range(2)]
    kd = [torch.empty_like(k[0]) for _ in range(2)]
    vd = [torch.empty_like(v[0]) for _ in range(2)]
    yd = [torch.empty(Bd, 1, H * DV, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    Ke = min(K, 400)
    main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_k = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def upload(i):
        b = i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_k[b])          # the kernel that last read these buffers has finished
            qd[b].copy_(qp[i % pool], non_blocking=True)
            kd[b].copy_(kp[i % pool], non_blocking=True)
            vd[b].copy_(vp[i % pool], non_blocking=True)
            ev_in[b].record(s_in)

    def e2e_loop(n):
        for b in range(2):
            ev_k[b].record(main); ev_out[b].record(s_out)
        upload(0)
        for i in range(n):
            b = i & 1
            if i + 1 < n:
                upload(i + 1)
            main.wait_event(ev_in[b])
            main.wait_event(ev_out[b])        # y buffer b has been copied out
            ops.linattn_decode(qd[b], kd[b], vd[b], kv, ks, out=yd[b])
            ev_k[b].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_k[b])
                yh[b].copy_(yd[b], non_blocking=True)
                ev_out[b].record(s_out)
        main.wait_stream(s_out)

    e2e_loop(4)
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    e2e_loop(Ke)
    f1.record()
    barrier()
    ms_e2e = f0.elapsed_time(f1)
    assert torch.isfinite(yh[0].float()).all() and torch.isfinite(yh[1].float()).all()

    from based_b200.sharding import max_over_ranks
    ms, ms_e2e = max_over_ranks([ms, ms_e2e], dev)

    if rank == 0:
        launch_ms = ms / K
        achieved = DEC_BYTES_PER_UNIT * Bd * H / (launch_ms * 1e-3) / 1e9
        line = {
            "metric": "decode_tok_per_s", "value": world * Bd * K / (ms * 1e-3), "unit": "tok/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": launch_ms, "higher_is_better": True,
            "scaling": "strong" if args.strong else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "decode microbench: B=256,H=16,d=16,dv=64, fp32 state [B,H,1,64,273], bf16 q/k/v, "
                                   "1 token/step; " + ("one batch split across the GPUs" if args.strong else "per-GPU shard fixed")
                                   + " (batch x heads), no collective",
                       "l2": "state (286 MB) larger than L2 (126 MB): no flush needed"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "traffic": None, "peak_source": peaks["source"],
                         "kernel": "linattn_decode_kernel<bf16,float>",
                         "algorithmic_bytes_per_launch": DEC_BYTES_PER_UNIT * Bd * H},
            "e2e": {"value": world * Bd * Ke / (ms_e2e * 1e-3), "unit": "tok/s",
                    "h2d_bytes_per_step": (qp[0].numel() + kp[0].numel() + vp[0].numel()) * 2,
                    "d2h_bytes_per_step": yh[0].numel() * 2, "steps": Ke},
            "gpu_launches": K,
            "clocks": clocks,
        }
        # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel at this size, from the ncu
        # capture summarised in profiles/linattn_decode_B256_H16.md (291.5 MB + 233.0 MB)
        line["roofline"]["traffic"] = 524.5e6
        if world == 1 and not args.no_sweep:
            lengths = args.sweep_L if args.sweep_L else ([2048] if args.quick else [2048, 8192, 32768])
            lin, swa = prefill_sweep(ops, peaks, lengths)
            line["prefill"] = lin
            line["swa"] = swa
            line["prefill_small_batch"] = small_batch_prefill(ops, max(lengths))
            line["gated_conv"] = gated_conv_bench(ops, peaks)
            line["norm_act"] = norm_act_bench(ops, peaks)
            if not args.quick:
                line["generation_360m"] = generation_bench()
                # the per-GPU share of the 8-GPU generation config: 8 of 64 sequences, prompt 4096, 1024 new tokens
                line["generation_1b"] = generation_bench(B=8, L=4096, new_tokens=1024, size="1b")
        if world == 1 and not args.no_cpu:
            use_all_host_threads()
            tput, dt = cpu_decode_baseline(B_DEC, 20, 2)
            line["cpu_baseline"] = {"value": tput, "unit": "tok/s", "cores": torch.get_num_threads(), "kind": "port",
                                    "sample": "20 full-batch recurrent steps (B=256,H=16) of the CPU restatement of "
                                              "recurrent_forward", "host_cpus": os.cpu_count()}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
