"""Benchmark of the Based hot path on B200.

Headline (the JSON line's ``value``): decode tok/s of the recurrent linear-attention step on
the decode microbench workload — bf16 q/k/v, fp32 state [B=256, H=16, 1, 64, 273], one token
per sequence per step.  One "step" is one pass of the decode kernel over the whole batch.
Per-GPU work is fixed as GPUs are added (batch x heads shards, no collective): weak scaling.

The same line carries: ``roofline`` (HBM fraction of the decode kernel), ``repeats`` (the timed region
run again many times: median / min / max and, with several GPUs, per-rank times), ``e2e`` (the same
step through the public API with host buffers: H2D of q/k/v and D2H of y inside the timed region),
``prefill`` / ``swa`` (the prefill sweep: tok/s and roofline fractions, each rank its own copy),
``cpu_baseline`` plus ``prefill_cpu`` / ``swa_cpu`` (the reference's own PyTorch code on the host cores,
one GPU only), ``generation_*`` (whole-model prompt pass and CUDA-graph decode), with several GPUs
``strong`` (the one batch split across the ranks) and ``tp`` (head-sharded mixers with the all-reduce after
the output projection), ``clocks`` sampled during the timed region and ``status`` (the kernels' bounded-wait
status word, 0 = no wait ever expired).

``--impl reference`` times the reference's own ``recurrent_forward`` (its unmodified Python module staged under
``oracle/_ref``; the CPU restatement of it when nothing is staged) on the host cores at the same B=256 workload,
and, when a GPU is visible, adds ``torch_on_gpu``: the same reference PyTorch code run on the GPU, so that a
GPU-against-GPU figure stands next to the CPU one.
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
# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the decode kernel at B=256, H=16 from an ncu capture
# (291.5 MB read + 233.0 MB written; the tail of the writes is still in L2 when the kernel ends)
DECODE_DRAM_TRAFFIC_PER_LAUNCH = 524.5e6
WORKLOAD = ("decode microbench: B=256,H=16,d=16,dv=64, fp32 state [B,H,1,64,273], bf16 q/k/v, "
            "1 token/step")


def workload_config(strong):
    """The `config` object of the JSON line; the same for both arms (they run the same workload)."""
    return {"workload": WORKLOAD,
            "sharding": ("one batch split across the GPUs" if strong else "per-GPU shard fixed") + " (batch x heads), no collective",
            "l2": "state (286 MB) larger than L2 (126 MB): no flush needed"}


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


def _reference_modules():
    """The reference's own LinearAttention / TaylorExp (staged copy), or None when nothing is staged."""
    try:
        from oracle import ref_shims
        if ref_shims.available():
            return ref_shims.reference(model=False)
    except Exception as exc:  # an import problem on this machine: fall back to the restatement, and say so
        print(f"[bench] staged reference not importable: {exc!r}", file=sys.stderr)
    return None


def _reference_mixer(ns, device="cpu"):
    m = ns.LinearAttention(d_model=H * DV, feature_map=ns.TaylorExp(input_dim=D_FEAT), feature_dim=D_FEAT,
                           num_heads=H, head_dim=DV)
    m.out_proj = torch.nn.Identity()
    return m.to(device)


def reference_decode(B, steps, warmup, device="cpu", seed=0):
    """tok/s of the reference's decode step (TaylorExp on q and k, then recurrent_forward,
    linear_attention.py:139, :230-251; out_proj = identity) at batch B on `device`.  Uses the staged reference
    module when present (kind "reference"), else the CPU restatement (kind "port")."""
    q, k, v, kv, ks = decode_inputs(B, 4, "cpu", seed)
    q, k, v = q.unsqueeze(3).to(device), k.unsqueeze(3).to(device), v.unsqueeze(3).to(device)   # [pool, B, H, 1, .]
    kv, ks = kv.to(device), ks.to(device)
    ns = _reference_modules()
    if ns is not None:
        m = _reference_mixer(ns, device)
        x = torch.zeros(B, 1, H * DV, device=device)

        def step(i):
            return m.recurrent_forward(x, kv, ks, m.feature_map(q[i % 4]), m.feature_map(k[i % 4]), v[i % 4])
        kind = "reference"
    else:
        from oracle import based_oracle as O

        def step(i):
            return O.linattn_recurrent_step(kv, ks, q[i % 4], k[i % 4], v[i % 4])
        kind = "port"
    sync = torch.cuda.synchronize if str(device).startswith("cuda") else (lambda: None)
    with torch.no_grad():
        for i in range(warmup):
            step(i)
        sync()
        t0 = time.perf_counter()
        for i in range(steps):
            step(i)
        sync()
        dt = time.perf_counter() - t0
    return B * steps / dt, dt, kind


def reference_prefill_cpu():
    """The reference's quadratic parallel_forward (linear_attention.py:171-183, :220-222) on the host cores:
    the parity configuration in full through LinearAttention.forward (d_model 1024, 16 heads, B=2, L=1024, fp32), and
    the prefill sweep's shapes on ONE (batch, head) slice each (the quadratic form needs B*H*L*L elements: 34 GB at
    L=8192 for the whole batch), scaled by B*H = 128 and labelled extrapolated."""
    ns = _reference_modules()
    if ns is None:
        return None
    out = {"kind": "reference", "cores": torch.get_num_threads()}
    with torch.no_grad():
        torch.manual_seed(0)
        m = ns.LinearAttention(d_model=1024, feature_map=ns.TaylorExp(input_dim=16), feature_dim=16, num_heads=16,
                               head_dim=64)
        x = torch.randn(2, 1024, 1024)
        m(x)
        t0 = time.perf_counter()
        for _ in range(3):
            m(x)
        dt = (time.perf_counter() - t0) / 3
        out["parity_config"] = {"shape": "B=2,L=1024,d_model=1024,H=16,fp32, whole mixer with projections",
                                "ms": dt * 1e3, "tok_per_s": 2 * 1024 / dt}
        mq = _reference_mixer(ns)
        mq.is_inference = True
        sweep = []
        for L in (2048, 8192):
            g = torch.Generator().manual_seed(L)
            q = torch.randn(1, 1, L, 16, generator=g) / 4
            k = torch.randn(1, 1, L, 16, generator=g) / 4
            v = torch.randn(1, 1, L, DV, generator=g) / 4
            xx = torch.zeros(1, L, DV)
            mq.num_heads = 1
            t0 = time.perf_counter()
            mq.parallel_forward(xx, q, k, v)
            dt = time.perf_counter() - t0
            sweep.append({"L": L, "slice_ms": dt * 1e3, "sample": "one (batch, head) slice of 128, fp32",
                          "tok_per_s_extrapolated": 8 * L / (dt * 8 * H)})
        out["sweep"] = sweep
        out["note"] = ("L=32768 is not run: one slice of the quadratic form needs 2 x 4.3 GB for A_qk alone; by the "
                       "measured L^2 growth it would be 16 x the L=8192 slice time")
    return out


def swa_restatement_cpu():
    """The reference has no CPU sliding-window attention (slide_attention.py:317-319: flash-attn only), so this
    times the CPU RESTATEMENT of its semantics on one (batch, head) slice of the sweep's shapes, scaled by B*H."""
    from oracle import based_oracle as O
    out = {"kind": "port", "cores": torch.get_num_threads(), "note": "CPU restatement of the reference's flash-attn "
           "call semantics, not reference code", "sweep": []}
    for L in (2048, 8192):
        g = torch.Generator().manual_seed(L)
        qkv = torch.randn(1, L, 3, 1, 64, generator=g) / 4
        t0 = time.perf_counter()
        O.swa_prefill(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], 64)
        dt = time.perf_counter() - t0
        out["sweep"].append({"L": L, "slice_ms": dt * 1e3, "sample": "one (batch, head) slice of 128, fp32",
                             "tok_per_s_extrapolated": 8 * L / (dt * 8 * H)})
    return out


def use_all_host_threads():
    """torchrun exports OMP_NUM_THREADS=1; the CPU legs are meant to use every host core."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(max(1, n))
    return n


def reference_on_gpu(steps):
    """The reference's own PyTorch code run on the GPU (what a user of the reference gets on this machine without
    this library): decode step at B=256 and the quadratic prefill at the sweep's shapes that fit."""
    ns = _reference_modules()
    if ns is None or not torch.cuda.is_available():
        return None
    out = {}
    tput, dt, kind = reference_decode(B_DEC, max(steps, 10), 3, device="cuda")
    out["decode"] = {"tok_per_s": tput, "ms_per_step": 1e3 * dt / max(steps, 10), "kind": kind,
                     "what": "TaylorExp x2 + recurrent_forward as torch ops on cuda, B=256, fp32 state, bf16 q/k/v"}
    m = _reference_mixer(ns, "cuda").bfloat16()
    m.is_inference = True
    pre = []
    with torch.no_grad():
        for L in (2048, 8192):
            g = torch.Generator(device="cuda").manual_seed(L)
            q = (torch.randn(8, H, L, 16, device="cuda", generator=g) / 4).bfloat16()
            k = (torch.randn(8, H, L, 16, device="cuda", generator=g) / 4).bfloat16()
            v = (torch.randn(8, H, L, DV, device="cuda", generator=g) / 4).bfloat16()
            xx = torch.zeros(8, L, H * DV, device="cuda", dtype=torch.bfloat16)
            try:
                m.parallel_forward(xx, q, k, v)
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                for _ in range(3):
                    m.parallel_forward(xx, q, k, v)
                torch.cuda.synchronize()
                dt = (time.perf_counter() - t0) / 3
                pre.append({"L": L, "ms": dt * 1e3, "tok_per_s": 8 * L / dt})
            except torch.cuda.OutOfMemoryError:
                pre.append({"L": L, "ms": None, "note": "out of memory (quadratic form)"})
            torch.cuda.empty_cache()
    pre.append({"L": 32768, "ms": None, "note": "not run: A_qk alone is 275 GB in bf16"})
    out["prefill_quadratic"] = pre
    return out


def run_reference(args, rank, world):
    if rank != 0:
        return
    use_all_host_threads()
    tput, dt, kind = reference_decode(B_DEC, args.steps, args.warmup)
    cores = torch.get_num_threads()
    what = ("the reference's own LinearAttention.recurrent_forward + TaylorExp (unmodified module, staged copy)"
            if kind == "reference" else "CPU restatement of recurrent_forward (no staged reference on this machine)")
    sample = (f"each step = one full recurrent step of the workload (B=256, H=16, fp32 state, bf16 q/k/v), "
              f"{args.steps} steps after {args.warmup} warm-up steps; {what}")
    line = {
        "impl": "reference", "metric": "decode_tok_per_s", "value": tput, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(False),
        "cpu_baseline": {"value": tput, "unit": "tok/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": tput, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "host_cpus": os.cpu_count(),
    }
    try:
        line["torch_on_gpu"] = reference_on_gpu(args.steps)
    except Exception as exc:  # the CPU figure above is the arm's result; this is an extra
        line["torch_on_gpu"] = {"error": repr(exc)}
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


def time_flushed(fn, flush, iters, warmup=3):
    """Device time per call of `fn` with L2 flushed before every call: the events sit between the flush and the
    kernel (flush -> event -> kernel -> event), and the per-call times are summed, so the flush itself is never in
    the measured interval.  The flush is long enough (256 MB of writes) that the host has queued the kernel and
    both events well before the first event is reached."""
    for _ in range(warmup):
        flush.zero_()
        fn()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for e0, e1 in ev:
        flush.zero_()
        e0.record()
        fn()
        e1.record()
    torch.cuda.synchronize()
    ts = sorted(e0.elapsed_time(e1) for e0, e1 in ev)
    return sum(ts) / len(ts), ts[0], ts[-1]  # ms: mean, min, max


def prefill_sweep(ops, peaks, lengths, dev):
    """Prefill sweep: B=8, H=16, d=16, dv=64, bf16, q/k/v ~ N(0,1)/4; linear attention and window-64 SWA.  With
    several GPUs every rank runs the whole sweep on its own copy (weak scaling); times are the max over ranks."""
    from based_b200.sharding import max_over_ranks
    out_lin, out_swa = [], []
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    for L in lengths:
        g = torch.Generator(device=dev).manual_seed(L)
        q = (torch.randn(8, H, L, 16, device=dev, generator=g) / 4).bfloat16()
        k = (torch.randn(8, H, L, 16, device=dev, generator=g) / 4).bfloat16()
        v = (torch.randn(8, H, L, DV, device=dev, generator=g) / 4).bfloat16()
        y = torch.empty(8, L, H, DV, dtype=torch.bfloat16, device=dev).permute(0, 2, 1, 3)
        kv = torch.empty(8, H, 1, DV, D_EXP, device=dev)
        ks = torch.empty(8, H, 1, 1, D_EXP, device=dev)
        iters = 10 if L >= 32768 else 20
        t, tmin, tmax = time_flushed(lambda: ops.linattn_prefill(q, k, v, out=y, kv_state=kv, k_state=ks), flush, iters)
        t, tmin, tmax = max_over_ranks([t, tmin, tmax], dev)
        units = 8 * H * L
        out_lin.append({"L": L, "ms": t, "ms_min": tmin, "ms_max": tmax, "tok_per_s": world * 8 * L / (t * 1e-3),
                        "tensor_frac": units * PREFILL_FLOP_PER_TOKEN_HEAD / (t * 1e-3) / (peaks["bf16_tflops"] * 1e12),
                        "hbm_frac": units * PREFILL_BYTES_PER_TOKEN_HEAD / (t * 1e-3) / (peaks["hbm_gbs"] * 1e9)})
        qkv = (torch.randn(8, L, 3, H, 64, device=dev, generator=g) / 4).bfloat16()
        o = torch.empty(8, L, H, 64, dtype=torch.bfloat16, device=dev)
        t, tmin, tmax = time_flushed(lambda: ops.swa_prefill(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], 64, out=o), flush,
                                     iters)
        t, tmin, tmax = max_over_ranks([t, tmin, tmax], dev)
        out_swa.append({"L": L, "ms": t, "ms_min": tmin, "ms_max": tmax, "tok_per_s": world * 8 * L / (t * 1e-3),
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
    from based_b200.sharding import max_over_ranks
    world = int(os.environ.get("WORLD_SIZE", "1"))
    pre_ms, dec_ms = max_over_ranks([t["prefill_ms"], t["decode_ms"]], ids.device)   # slowest rank
    res = {"model": f"based-{size} (random init)", "params": nparam, "B_per_gpu": B, "B_total": world * B, "prompt": L,
           "new_tokens": new_tokens, "sharding": "batch-sharded replicas, no communication",
           "prefill_ms": pre_ms, "prefill_tok_per_s": world * B * L / (pre_ms * 1e-3),
           "decode_ms_per_step": dec_ms / steps, "decode_tok_per_s": world * B * steps / (dec_ms * 1e-3),
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


def tp_bench(dev, world):
    """The tensor-parallel variant of the 8-GPU generation configuration: the 1.4B model's LinearAttention and
    SlidingAttention mixers (d_model 1792, 16 heads, head_dim 112) head-sharded over the ranks — q/k/v projections
    column-parallel, state / KV cache local, out_proj row-parallel, ONE all-reduce of [B, L, d_model] at the end
    (modelled on RowParallelLinear.forward, based/ops/fused_dense.py:239-246).  Activations are replicated, so every
    rank sees the whole batch of 64.  Times are CUDA-event device times, max over ranks; `allreduce_ms` is the same
    collective on a tensor of the output's size timed on its own, `allreduce_share` its part of the mixer's time."""
    import torch.distributed as dist
    from based_b200.generation import InferenceParams
    from based_b200.mixers import LinearAttention, SlidingAttention, TaylorExp
    from based_b200.sharding import max_over_ranks
    Dm, Hh, B, L = 1792, 16, 64, 4096
    if Hh % world != 0:
        return None
    torch.manual_seed(0)
    kw = {"device": dev, "dtype": torch.bfloat16, "process_group": dist.group.WORLD}
    mixers = {
        "linear_attention": LinearAttention(Dm, feature_map=TaylorExp(16), num_heads=Hh, layer_idx=0, fuse_qkv=True, **kw),
        "sliding_attention": SlidingAttention(Dm, Hh, qkv_proj_bias=False, out_proj_bias=False, rotary_emb_dim=Dm // Hh,
                                              window_size=128, layer_idx=1, **kw),
    }
    x = torch.randn(B, L, Dm, device=dev, dtype=torch.bfloat16)
    x1 = torch.randn(B, 1, Dm, device=dev, dtype=torch.bfloat16)

    def timed(fn, iters):
        for _ in range(2):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return max_over_ranks([e0.elapsed_time(e1) / iters], dev)[0]

    out = {"config": f"d_model={Dm}, heads={Hh} ({Hh // world} per rank), head_dim={Dm // Hh}, B={B}, prompt={L}, bf16, "
                     "NCCL all-reduce after out_proj"}
    buf_p = torch.empty(B, L, Dm, device=dev, dtype=torch.bfloat16)
    buf_d = torch.empty(B, 1, Dm, device=dev, dtype=torch.bfloat16)
    ar_p = timed(lambda: dist.all_reduce(buf_p), 5)
    ar_d = timed(lambda: dist.all_reduce(buf_d), 50)
    out["allreduce_prompt_ms"], out["allreduce_prompt_bytes"] = ar_p, buf_p.numel() * 2
    out["allreduce_decode_ms"], out["allreduce_decode_bytes"] = ar_d, buf_d.numel() * 2
    with torch.inference_mode():
        for name, m in mixers.items():
            m.eval()
            ip = InferenceParams(max_seqlen=L + 64, max_batch_size=B)
            ip.key_value_memory_dict[m.layer_idx] = m.allocate_inference_cache(B, L + 64, dtype=torch.bfloat16)
            ip.lengths_per_sample = torch.full((B,), L, dtype=torch.int32, device=dev)

            def prompt():
                ip.seqlen_offset = 0
                m(x, inference_params=ip)

            def step():
                ip.seqlen_offset = L
                m(x1, inference_params=ip)

            tp_ms = timed(prompt, 5)
            td_ms = timed(step, 50)
            out[name] = {"prompt_ms": tp_ms, "prompt_tok_per_s": B * L / (tp_ms * 1e-3),
                         "prompt_allreduce_share": ar_p / tp_ms,
                         "decode_step_ms": td_ms, "decode_tok_per_s": B / (td_ms * 1e-3),
                         "decode_allreduce_share": ar_d / td_ms, "decode_timing": "eager launches, device time"}
            # the same step with out_proj and the all-reduce as ONE kernel per rank (partial tiles pushed through peer
            # memory); the output projection + collective alone, both ways, captured in CUDA graphs of 20 calls
            try:
                m.fused_allreduce = True
                step()                                    # builds the peer workspace (a collective)
                out[name]["decode_step_fused_ms"] = timed(step, 50)
                from based_b200.sharding import all_reduce_sum_
                yl = torch.randn(B, 1, m.out_proj.weight.shape[1], device=dev, dtype=torch.bfloat16)
                w = m.out_proj.weight
                fused = m._fused_row_parallel
                t_f = max_over_ranks([time_graph(lambda: fused(yl, w), 20)], dev)[0]
                t_n = max_over_ranks([time_graph(lambda: all_reduce_sum_(torch.nn.functional.linear(yl, w),
                                                                       dist.group.WORLD), 20)], dev)[0]
                out[name]["outproj_allreduce_fused_us"] = t_f * 1e3
                out[name]["outproj_allreduce_cublas_nccl_us"] = t_n * 1e3
            except Exception as exc:   # peer mapping unavailable on this machine: the NCCL figures above stand
                out[name]["fused_error"] = repr(exc)
            finally:
                m.fused_allreduce = False
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--strong", action="store_true",
                    help="strong scaling: split the one B=256 batch across the GPUs instead of one batch per GPU")
    ap.add_argument("--no-sweep", action="store_true", help="skip the prefill / SWA sweep and the model runs")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline legs")
    ap.add_argument("--quick", action="store_true", help="prefill sweep at L=2048 only, no model runs")
    ap.add_argument("--sweep-L", type=int, nargs="*", default=None, help="sequence lengths of the prefill sweep")
    ap.add_argument("--regions", type=int, default=25, help="how many times the K-step region is repeated for the "
                    "median / min / max record (the first one is the headline)")
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
    from based_b200.sharding import max_over_ranks
    build_library()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()
    K, W, pool = args.steps, args.warmup, 16
    PREROLL = 2000  # untimed steps before the warm-up (0.2 s): brings clocks and caches to their loaded state

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def decode_region(Bd, seed, regions):
        """W warm-up steps, then `regions` timed regions of exactly K steps each (the first one bracketed by a barrier
        and a synchronize on both sides).  Returns the per-region times in ms and the clock record of the first."""
        qh, kh, vh, kv0, ks0 = decode_inputs(Bd, pool, "cpu", seed=seed)
        q, k, v = qh.to(dev), kh.to(dev), vh.to(dev)
        kv, ks = kv0.to(dev), ks0.to(dev)
        y = torch.empty(Bd, 1, H * DV, dtype=torch.bfloat16, device=dev)

        def steps(n):
            for i in range(n):
                ops.linattn_decode(q[i % pool], k[i % pool], v[i % pool], kv, ks, out=y)

        # The clock sampler (a child process) is started BEFORE the untimed steps, so that nothing but the barrier
        # and the synchronize stands between the warm-up and the timed region: a GPU left idle while a process is
        # spawned starts the region from its idle state, which a 2 ms region feels.
        sampler = ClockSampler(local_rank) if rank == 0 else None
        if sampler:
            sampler.start()
        # With several ranks, a barrier BEFORE the untimed steps lines the ranks up (their start-up times differ by
        # seconds), so that the barrier in front of the timed region is a short wait and not a long idle period on
        # the ranks that came first.
        barrier()
        # The untimed steps are drained in slices: with a thousand launches queued ahead of the GPU, the first
        # region after them measured 3-8 % slower than the following ones (and than after a drained pre-roll).
        for _ in range(PREROLL // 200):
            steps(200)
            torch.cuda.synchronize()
        steps(W)
        barrier()
        times = []
        for r in range(regions):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            steps(K)
            e1.record()
            barrier()
            times.append(e0.elapsed_time(e1))
            if r == 0 and sampler:
                clocks = sampler.stop()
        assert torch.isfinite(y.float()).all()
        return times, (clocks if rank == 0 else None), (qh, kh, vh, q, k, v, kv, ks)

    # ---------------- device-resident timed region (weak scaling: every rank its own B=256 batch) ----------------
    Bd = B_DEC // world if args.strong else B_DEC
    times, clocks, (qh, kh, vh, q, k, v, kv, ks) = decode_region(Bd, rank, max(1, args.regions))
    ms = times[0]
    srt = sorted(times)
    rep_local = [srt[len(srt) // 2] / K, srt[0] / K, srt[-1] / K]
    if world > 1:
        allr = [None] * world
        dist.all_gather_object(allr, rep_local)
    else:
        allr = [rep_local]

    # ---------------- end to end: host buffers, H2D + kernel + D2H per step ----------------
    # Every step copies its q/k/v from pinned host memory and returns y to pinned host memory through
    # the public op.  The copies run on their own streams, double-buffered, so that step i+1's inputs
    # travel while step i computes (what a serving loop does); the state stays on the device.
    # q, k and v of a step sit back to back in ONE pinned buffer and land in one device buffer, so a step's inputs
    # are one copy (786 KB) instead of three; the op gets views of that buffer.
    nq, nk, nv = qh[0].numel(), kh[0].numel(), vh[0].numel()
    inp = torch.cat([qh.reshape(pool, -1), kh.reshape(pool, -1), vh.reshape(pool, -1)], dim=1).contiguous().pin_memory()
    yh = [torch.empty(Bd, 1, H * DV, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    ind = [torch.empty(nq + nk + nv, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    qd = [t[:nq].view_as(q[0]) for t in ind]
    kd = [t[nq:nq + nk].view_as(k[0]) for t in ind]
    vd = [t[nq + nk:].view_as(v[0]) for t in ind]
    yd = [torch.empty(Bd, 1, H * DV, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    # at least 200 steps, so that filling and draining the three-stage pipeline (upload, kernel, download) is not a
    # sixth of the measurement; the record carries its own step count
    Ke = min(max(K, 200), 400)
    main_s = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_k = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def upload(i):
        b = i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_k[b])          # the kernel that last read these buffers has finished
            ind[b].copy_(inp[i % pool], non_blocking=True)
            ev_in[b].record(s_in)

    def e2e_loop(n):
        for b in range(2):
            ev_k[b].record(main_s); ev_out[b].record(s_out)
        upload(0)
        for i in range(n):
            b = i & 1
            if i + 1 < n:
                upload(i + 1)
            main_s.wait_event(ev_in[b])
            main_s.wait_event(ev_out[b])        # y buffer b has been copied out
            ops.linattn_decode(qd[b], kd[b], vd[b], kv, ks, out=yd[b])
            ev_k[b].record(main_s)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_k[b])
                yh[b].copy_(yd[b], non_blocking=True)
                ev_out[b].record(s_out)
        main_s.wait_stream(s_out)

    e2e_loop(max(4, W))
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    e2e_loop(Ke)
    f1.record()
    barrier()
    ms_e2e = f0.elapsed_time(f1)
    assert torch.isfinite(yh[0].float()).all() and torch.isfinite(yh[1].float()).all()
    ms, ms_e2e = max_over_ranks([ms, ms_e2e], dev)
    h2d = inp[0].numel() * 2
    d2h = yh[0].numel() * 2
    del inp, ind, q, k, v, kv, ks

    line = None
    if rank == 0:
        launch_ms = ms / K
        achieved = DEC_BYTES_PER_UNIT * Bd * H / (launch_ms * 1e-3) / 1e9
        med = max(a[0] for a in allr)
        line = {
            "metric": "decode_tok_per_s", "value": world * Bd * K / (ms * 1e-3), "unit": "tok/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": launch_ms, "higher_is_better": True,
            "scaling": "strong" if args.strong else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args.strong), "preroll_steps": PREROLL,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "traffic": DECODE_DRAM_TRAFFIC_PER_LAUNCH,
                         "peak_source": peaks["source"], "kernel": "linattn_decode_kernel<bf16,float>",
                         "algorithmic_bytes_per_launch": DEC_BYTES_PER_UNIT * Bd * H},
            "repeats": {"regions": len(times), "steps_per_region": K, "what": "the same K-step region run again; "
                        "ms per step, slowest rank's median, and every rank's (median, min, max)",
                        "ms_per_step_median": med, "frac_at_median": DEC_BYTES_PER_UNIT * Bd * H / (med * 1e-3) / 1e9 / peaks["hbm_gbs"],
                        "per_rank_ms_per_step": allr,
                        "first_regions_ms_per_step": [t / K for t in times[:6]]},
            "e2e": {"value": world * Bd * Ke / (ms_e2e * 1e-3), "unit": "tok/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": Ke},
            "gpu_launches": K,
            "clocks": clocks,
        }

    # ---------------- extra records (every rank takes part; rank 0 keeps the results) ----------------
    extras = {}
    if not args.no_sweep:
        lengths = args.sweep_L if args.sweep_L else ([2048] if args.quick else [2048, 8192, 32768])
        lin, swa = prefill_sweep(ops, peaks, lengths, dev)
        extras["prefill"], extras["swa"] = lin, swa
        if world == 1:
            extras["prefill_small_batch"] = small_batch_prefill(ops, max(lengths))
            extras["gated_conv"] = gated_conv_bench(ops, peaks)
            extras["norm_act"] = norm_act_bench(ops, peaks)
        if world > 1 and not args.strong:
            # strong scaling: the ONE B=256 batch split across the ranks
            st, _, _ = decode_region(B_DEC // world, 100 + rank, 5)
            st_ms = max_over_ranks([sorted(st)[len(st) // 2]], dev)[0]
            extras["strong"] = {"B_per_gpu": B_DEC // world, "ms_per_step": st_ms / K,
                                "tok_per_s": B_DEC * K / (st_ms * 1e-3), "what": "median of 5 regions, slowest rank"}
        if not args.quick:
            if world == 1:
                extras["generation_360m"] = generation_bench()
            # 8 sequences per GPU, prompt 4096, 1024 new tokens: with 8 GPUs this is the 64-sequence generation config
            extras["generation_1b"] = generation_bench(B=8, L=4096, new_tokens=1024, size="1b")
            if world > 1:
                extras["tp"] = tp_bench(dev, world)
    torch.cuda.synchronize()
    status = ops.check_status()   # raises if any tensor-core kernel gave up on a bounded wait

    if rank == 0:
        line.update(extras)
        line["status"] = status
        if world == 1 and not args.no_cpu:
            use_all_host_threads()
            tput, dt, kind = reference_decode(B_DEC, 20, 2)
            line["cpu_baseline"] = {"value": tput, "unit": "tok/s", "cores": torch.get_num_threads(), "kind": kind,
                                    "sample": "20 full-batch recurrent steps (B=256,H=16) of the reference's "
                                              "recurrent_forward on the host cores" if kind == "reference" else
                                              "20 full-batch recurrent steps of the CPU restatement of recurrent_forward",
                                    "host_cpus": os.cpu_count()}
            if not args.quick:
                line["prefill_cpu"] = reference_prefill_cpu()
                line["swa_cpu"] = swa_restatement_cpu()
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
