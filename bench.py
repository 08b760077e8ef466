#!/usr/bin/env python
"""Benchmark of the attention hot path: Nikhilam INT8-KV decode attention at 8K context.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (one "step" = one decode step over the whole batch): 64 sequences, 16 heads,
DH 64, 8191 cached tokens + the new token; K/V pre-quantization values ~ N(0,1) with 1 %
outliers x8, quantized with one scale per (sequence, head, K|V) tensor; Q in FP16; the new
token is quantized on append, then attention streams the INT8 cache.  Heads are sharded
over the GPUs (total work fixed: strong scaling) and every rank ends the step with the
gathered [B][H][DH] output (the engine's peer-memory exchange; no library collective).

Prints ONE JSON line.  At every N the step is replayed as one CUDA graph per step; the
`steps` loop is repeated several times and the median repeat is reported.
  value      device-resident step, CUDA events around the loop, max over ranks
  roofline   decode_dense_kernel alone, replayed the same way over the same rotating caches
  e2e        the step through host buffers: copies in and out and a synchronisation per step
  secondary  the prefill and Shunyam-window kernels, each checked against the CPU oracle on sampled rows
  baselines  (one GPU only) the reference's CPU forward of configuration 1 and the reference's own
             CUDA kernels timed on this GPU beside the engine's on the same inputs
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

B, H, S_MAX, DH = 64, 16, 8192, 64
ETA, NU = 0.1, 0.05
REPEATS = 7      # the `steps` loop is timed this many times; the median is reported
# DRAM bytes that one (sequence, head) pair of decode_dense_kernel moves at 8192 cached tokens,
# from a hardware-counter capture of a 256-pair launch (268.55 MB read + 4.20 MB written).  Pairs are
# independent, so a launch moves this times its number of pairs.
DECODE_TRAFFIC_PER_PAIR = (268.55e6 + 4.20e6) / 256
L_OPT_WORKSPACE_LOCK = 3            # logos_option of include/logos_attn.h
METRIC = "int8_kv_decode_attention_bandwidth_8k_ctx"
UNIT = "GB/s"


def workload_config(world: int) -> dict:
    """What is computed -- the same dictionary in both arms."""
    return {"workload": f"int8_kv_decode_b{B}_h{H}_ctx{S_MAX}_dh{DH}", "batch": B, "heads": H, "ctx": S_MAX, "dh": DH,
            "ns_eta": ETA, "ns_nu": NU, "diffusion": "causal", "parallelism": f"heads/{world}"}


def algorithmic_bytes(b: int, h: int, s: int, dh: int) -> int:
    """INT8 K + V read once, plus scales, Q/q_prev, the output and the appended rows."""
    return 2 * b * h * s * dh + 2 * b * h * 4 + 2 * b * h * dh * 2 + b * h * dh * 4 + 2 * b * h * dh


def measured_peaks() -> dict:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            j = json.load(f)
        return {"hbm": float(j["hbm_gbs"]), "tensor": float(j["bf16_tflops"]), "kind": "measured"}
    except Exception:
        return {"hbm": 6650.0, "tensor": 1590.0, "kind": "fallback"}


def median(xs):
    xs = sorted(xs)
    return xs[len(xs) // 2]


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-lms", "50", "-i", str(self.idx)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def stop(self) -> dict:
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except Exception:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.f.read().splitlines():
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1])); mx.append(float(c[2]))
            except ValueError:
                continue
            for n, v in zip(names, c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        os.unlink(self.f.name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------------
# CPU legs (test infrastructure under oracle/ is executed only here)

def cpu_port_baseline(sample_pairs: int = 128) -> dict:
    """The CPU oracle's decode (same arithmetic, row-only, OpenMP over pairs) on a bounded
    sample of the workload: `sample_pairs` of the 1024 (sequence, head) pairs at full context."""
    import numpy as np
    import oracle as O
    rng = np.random.default_rng(0)
    n = sample_pairs
    kq = rng.integers(-127, 128, (n, S_MAX, DH), dtype=np.int8)
    vq = rng.integers(-127, 128, (n, S_MAX, DH), dtype=np.int8)
    q = rng.standard_normal((n, DH)).astype(np.float32)
    qp = rng.standard_normal((n, DH)).astype(np.float32)
    sc = np.full(n, 0.03, np.float32)
    lens = np.full(n, S_MAX, np.int32)
    p = O.attn_params(0.125, True, 0, 0, ETA, NU, 1.0, O.DIFFUSE_CAUSAL)
    threads = O.lib().lo_max_threads()
    O.decode_int8_batch(q[:threads], qp[:threads], kq[:threads], vq[:threads], sc[:threads], sc[:threads],
                        lens[:threads], p, threads)  # warm the thread pool
    reps, t0 = 0, time.perf_counter()
    while True:
        O.decode_int8_batch(q, qp, kq, vq, sc, sc, lens, p, threads)
        reps += 1
        dt = time.perf_counter() - t0
        if dt > 10.0 or reps >= 50:
            break
    gbs = reps * algorithmic_bytes(1, n, S_MAX, DH) / dt / 1e9
    return {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{n} of {B * H} (sequence, head) pairs at ctx {S_MAX}, {reps} passes, "
                      "CPU oracle reading only the decode row"}


def configuration1_cpu_baseline() -> dict:
    """The reference's MultiHeadAttention::forward (include/Attention.hpp:290-300) at benchmark
    configuration 1 (seq 512, d_model 1024, 16 heads, causal, Navier-Stokes on), compiled unmodified
    with the reference's flags (-O3 -march=x86-64, CMakeLists.txt:39) and with -march=x86-64-v3, on
    one thread (as the reference runs) and with the heads farmed over all host threads."""
    import ctypes as C
    import numpy as np
    import oracle as O
    from logos_b200 import synthetic as syn
    seq, d, heads = 512, 1024, 16
    dk = d // heads
    X = syn.normal((seq, d), 1, 1)
    W = [syn.normal(s, 1, t, std=0.02) for t, s in enumerate(
        [(heads, d, dk), (heads, d, dk), (heads, d, dk), (heads, dk, d), (d, d)], start=2)]
    out = np.empty((seq, d), np.float32)
    res = {"config": "seq 512, d_model 1024, H 16, DH 64, fp32, causal, NS alpha 1 eta 0.1 nu 0.05",
           "gflop": 2 * 512 * 1024 * 64 * 3 * 16 / 1e9 + 4 * 512 * 512 * 64 * 16 * 2 / 1e9 +
                    2 * 512 * 64 * 1024 * 16 / 1e9 + 2 * 512 * 1024 * 1024 / 1e9, "runs": []}
    for flags, R in (("-O3 -march=x86-64", O.ref()), ("-O3 -march=x86-64-v3", O.ref_v3())):
        if R is None:
            res["runs"].append({"flags": flags, "unavailable": "not built, or this host lacks the instruction set"})
            continue
        nthreads = max(1, min(R.ref_hardware_threads(), heads))
        for threads in (1, nthreads):
            cfg = O.HeadCfg(0, 8, 4, 1, 1.0, ETA, NU, 0, threads)
            R.ref_mha_forward(X, *W, seq, d, heads, C.byref(cfg), out)       # warms the mask cache
            t0 = time.perf_counter()
            R.ref_mha_forward(X, *W, seq, d, heads, C.byref(cfg), out)
            res["runs"].append({"flags": flags, "threads": threads, "ms_per_forward": (time.perf_counter() - t0) * 1e3})
    res["nproc"] = os.cpu_count()
    return res


def run_reference(args) -> None:
    """The reference's own CPU attention (include/Attention.hpp, compiled unmodified) doing what
    a decode step costs in the reference today: a full re-forward of every (sequence, head)
    over its whole context (cuda/train_gpu.cu:2037-2046), heads farmed over all host threads.
    Each step is a bounded sample: one pair per thread at the full 8192-token context.  This is
    the reference's real cost per token, not a kernel comparison: the algorithmically equal CPU
    number is `cpu_baseline` of the other arm."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import ctypes as C
    import numpy as np
    import oracle as O
    R = O.ref()
    world = args.gpus
    base = {"impl": "reference", "metric": METRIC, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": True}
    if R is None:
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref was not built (reference tree absent at build time)"}))
        return
    R.ref_ns_attention_batch.argtypes = [O.f32p, O.f32p, O.f32p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float,
                                         O.f32p, C.c_int]
    threads = max(1, min(R.ref_hardware_threads(), 32))
    n = threads
    rng = np.random.default_rng(0)
    # dequantized K/V of the sample pairs (the reference attends over fp32 K/V) and a full Q
    kq = rng.integers(-127, 128, (n, S_MAX, DH), dtype=np.int8)
    vq = rng.integers(-127, 128, (n, S_MAX, DH), dtype=np.int8)
    K = (kq.astype(np.float32) * np.float32(0.03))
    V = (vq.astype(np.float32) * np.float32(0.03))
    Q = rng.standard_normal((n, S_MAX, DH)).astype(np.float32)
    out = np.empty_like(Q)
    for _ in range(args.warmup):
        R.ref_ns_attention_batch(Q, K, V, n, S_MAX, DH, ETA, NU, out, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        R.ref_ns_attention_batch(Q, K, V, n, S_MAX, DH, ETA, NU, out, threads)
    dt = (time.perf_counter() - t0) / max(args.steps, 1)
    gbs = algorithmic_bytes(1, n, S_MAX, DH) / dt / 1e9
    sample = (f"{n} of {B * H} (sequence, head) pairs per step at ctx {S_MAX}, one per thread; "
              "navier_stokes_attention over the whole context (what a generated token costs the reference today), "
              "last row is the decode output")
    base.update({"value": gbs, "ms_per_step": dt * 1e3, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                 "data": "synthetic", "config": workload_config(world),
                 "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": threads, "kind": "reference", "sample": sample},
                 "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
    print(json.dumps(base))


# ---------------------------------------------------------------------------------------------
# the other kernels of the path

PREFILL = {"name": "causal_prefill_b4_h16_s4096_dh64_bf16", "B": 4, "S": 4096, "window": 0, "outliers": False}
PREFILL_8K = {"name": "causal_prefill_b4_h16_s8192_dh64_bf16", "B": 4, "S": 8192, "window": 0, "outliers": False}
WINDOW = {"name": "shunyam_window64_b8_h16_s8192_dh64_bf16", "B": 8, "S": 8192, "window": 64, "stride": 0,
          "outliers": True}
# the reference's production setting: window 64 plus every 16th key as a landmark (cuda/train_gpu.cu:1172-1173)
WINDOW_LM = {"name": "shunyam_window64_stride16_b8_h16_s8192_dh64_bf16", "B": 8, "S": 8192, "window": 64,
             "stride": 16, "outliers": True}


def check_against_oracle(Q, K, V, out, cfg) -> float:
    """Sampled heads and row ranges of a device result against the CPU oracle; max-abs error."""
    import numpy as np
    import oracle as O
    S = cfg["S"]
    op = O.attn_params(0.125, True, cfg["window"], cfg.get("stride", 0), ETA, NU, 1.0, O.DIFFUSE_CAUSAL)
    worst = 0.0
    heads = [(0, 0), (Q.shape[0] - 1, Q.shape[1] - 1)]
    for (b, h) in heads:
        q, k, v = (t[b, h].float().cpu().numpy() for t in (Q, K, V))
        for (r0, r1) in [(0, 66), (250, 262), (S // 2 - 3, S // 2 + 3), (S - 8, S)]:
            want = O.attention_rows(q, k, v, op, r0, r1)
            got = out[b, h, r0:r1].float().cpu().numpy()
            d = np.abs(got - want)
            worst = max(worst, float(d.max()) if np.isfinite(d).all() else float("inf"))
    return worst


def measure_attention(eng, dev, world, rank, cfg, steps, warmup, barrier, max_over_ranks, comm=None) -> dict:
    """Device-resident prefill / window attention over this rank's heads (BF16 in, BF16 out,
    Navier-Stokes prologue fused: eta 0.1, causal diffusion nu 0.05); with several GPUs the outputs
    are gathered through the engine's peer-memory exchange."""
    import torch
    from logos_b200 import lib as L
    from logos_b200.sharding import head_range
    lo, hi = head_range(H, rank, world)
    Hl, Bc, S = hi - lo, cfg["B"], cfg["S"]
    g = torch.Generator(device=dev).manual_seed(2000 + rank)
    sets = []
    for _ in range(2):   # two input sets in rotation: a pass never finds its inputs in L2
        Q, K, V = (torch.randn((Bc, Hl, S, DH), device=dev, generator=g) for _ in range(3))
        if cfg["outliers"]:
            K[torch.rand(K.shape, device=dev, generator=g) < 0.01] *= 8
        sets.append(tuple(t.bfloat16() for t in (Q, K, V)))
        del Q, K, V
    O = torch.empty((Bc, Hl, S, DH), dtype=torch.bfloat16, device=dev)
    gathered = torch.empty((Bc, H, S, DH), dtype=torch.bfloat16, device=dev) if world > 1 else None
    p = L.Params.make(1.0 / 8.0, True, cfg["window"], cfg.get("stride", 0), ETA, NU, 1.0, L.DIFFUSE_CAUSAL)

    def step(i):
        Q, K, V = sets[i % 2]
        eng.attention(Q, K, V, p, out=O)
        if world > 1:
            comm.all_gather_heads(O, gathered)

    for i in range(warmup):
        step(i)
    times = []
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    for _ in range(3):
        barrier()
        ev[0].record()
        for i in range(steps):
            step(warmup + i)
        ev[1].record()
        barrier()
        times.append(ev[0].elapsed_time(ev[1]) / steps)
    eng.synchronize()
    ms = max_over_ranks(median(times))
    # correctness of what was just timed, outside the timed region: the same call once more with fp32
    # output against the oracle (tolerance 2e-3), and the timed BF16 output must be its rounding
    Q, K, V = sets[(warmup + steps - 1) % 2]
    O32 = eng.attention(Q, K, V, p, out_dtype=torch.float32)
    eng.synchronize()
    err = max_over_ranks(check_against_oracle(Q, K, V, O32, cfg))
    same = bool(torch.equal(O32.bfloat16(), O))
    out = {"workload": cfg["name"], "ms_per_step": ms, "n_gpus": world, "max_abs_err_vs_oracle": err,
           "timed_output_is_the_bf16_rounding_of_the_checked_one": same,
           "checked": "two heads x four row ranges of the last timed step's inputs, fp32 output, tolerance 2e-3"}
    del O32
    peaks = measured_peaks()
    if cfg["window"]:
        nbytes = 4 * Bc * H * S * DH * 2                       # Q, K, V read once, O written once
        out.update({"value": nbytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "bound": "hbm", "peak": peaks["hbm"],
                    "peak_kind": peaks["kind"], "frac": nbytes / (ms * 1e-3) / 1e9 / (peaks["hbm"] * world)})
    else:
        flops = 4.0 * Bc * H * S * S * DH / 2                  # causal-halved convention
        out.update({"value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s (causal-halved)", "bound": "tensor",
                    "peak": peaks["tensor"], "peak_kind": peaks["kind"] + " burst",
                    "frac": flops / (ms * 1e-3) / 1e12 / (peaks["tensor"] * world)})
    return out


def measure_stack(eng, dev, world, rank, comm, barrier, max_over_ranks, layers=16, batch=32, prompt=2048, steps=128) -> dict:
    """Benchmark configuration 5: the 16-layer attention stack (d 1024, 16 heads, vocabulary 8192, weights
    ~ N(0, 0.02)), 32 prompts of 2048 uniform-random token ids prefilled into the INT8 cache, then 128
    decode steps with Shunyam window 64 / stride 16; heads sharded over the GPUs, per-head outputs gathered.
    Reports tokens/s of the decode phase, the time of each phase and the attention kernels' own share."""
    import torch
    from logos_b200.stack import AttentionStack, StackConfig, make_weights
    cfg = StackConfig(num_layers=layers, max_seq_len=prompt + steps)
    w = make_weights(cfg, seed=5, std=0.02, device=dev)
    st = AttentionStack(eng, cfg, w, batch=batch, rank=rank, world=world, comm=comm)
    del w
    g = torch.Generator(device=dev).manual_seed(5000)
    ids = torch.randint(0, cfg.vocab_size, (batch, prompt), device=dev, generator=g)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    st.prefill(ids)                                    # warm-up (lazy set-up, allocator)
    barrier()
    ev[0].record()
    logits = st.prefill(ids)
    ev[1].record()
    barrier()
    prefill_ms = max_over_ranks(ev[0].elapsed_time(ev[1]))
    graph, gids, glogits = st.capture_decode(greedy=True)     # the graph feeds its arg-max tokens back into gids
    gids.copy_(logits.argmax(dim=1))
    barrier()
    ev[0].record()
    for _ in range(steps):
        graph.replay()
    ev[1].record()
    barrier()
    decode_ms = max_over_ranks(ev[0].elapsed_time(ev[1]))
    finite = bool(torch.isfinite(glogits).all())
    # the attention kernels alone, on one layer's tensors
    Hl, S = st.Hl, prompt
    Q, K, V = (torch.randn((batch, Hl, S, DH), device=dev, generator=g).bfloat16() for _ in range(3))
    for _ in range(2):
        O = eng.attention(Q, K, V, st.params)
    ev[0].record()
    for _ in range(5):
        eng.attention(Q, K, V, st.params, out=O)
    ev[1].record()
    torch.cuda.synchronize()
    attn_ms = max_over_ranks(ev[0].elapsed_time(ev[1]) / 5)
    kc, vc, ks, vs = st.cache.layer(0)
    q = torch.randn((batch, Hl, DH), device=dev, generator=g).half()
    lens = st.cache.lens.clone()
    o = torch.empty((batch, Hl, DH), device=dev)
    for _ in range(3):
        eng.decode_int8(q, q, kc, vc, ks, vs, lens, st.params, out=o)
    ev[0].record()
    for _ in range(20):
        eng.decode_int8(q, q, kc, vc, ks, vs, lens, st.params, out=o)
    ev[1].record()
    torch.cuda.synchronize()
    dec_attn_ms = max_over_ranks(ev[0].elapsed_time(ev[1]) / 20)
    ctx = prompt + steps
    keys = min(ctx, cfg.window + 1) + max(0, (ctx - 1 - cfg.window + cfg.stride - 1) // cfg.stride)   # window + landmarks
    peaks = measured_peaks()
    graph.reset()
    eng.set_option(L_OPT_WORKSPACE_LOCK, 0)
    win_bytes = 4 * batch * cfg.num_heads * S * DH * 2
    return {"workload": f"stack_l{layers}_d1024_h16_b{batch}_prompt{prompt}_decode{steps}_window64_stride16",
            "n_gpus": world, "tokens_per_s_decode": batch * steps / (decode_ms * 1e-3),
            "tokens_per_s_prefill": batch * prompt / (prefill_ms * 1e-3),
            "prefill_ms": prefill_ms, "decode_ms_per_step": decode_ms / steps, "logits_finite": finite,
            "launch": "prefill eager, decode step replayed as one CUDA graph (all layers, the arg-max token fed back inside the graph)",
            "attention_only": {
                "prefill_attention_ms_per_layer": attn_ms,
                "prefill_attention_share_of_phase": attn_ms * layers / prefill_ms,
                "prefill_attention_gbs": win_bytes / world / (attn_ms * 1e-3) / 1e9,
                "prefill_attention_frac_of_hbm_peak": win_bytes / world / (attn_ms * 1e-3) / 1e9 / peaks["hbm"],
                "decode_attention_ms_per_layer": dec_attn_ms,
                "decode_attention_share_of_step": dec_attn_ms * layers / (decode_ms / steps),
                "decode_visible_keys_per_query_at_end": keys,
                "decode_attention_bytes_per_step_per_layer": batch * cfg.num_heads * keys * DH * 2,
                "note": "decode attention reads ~200 scattered rows per pair: latency-bound, not a bandwidth figure"}}


def measure_projection(eng, dev, batch, steps, warmup) -> dict:
    """The fused Q/K/V projection of configuration 5's prefill alone: [batch * 2048, 1024] x [1024, 3072] BF16
    with the scatter into [B][H][S][64] and the quantiser's max|x| in the epilogue."""
    import torch
    S, D, Hh = 2048, 1024, H
    g = torch.Generator(device=dev).manual_seed(77)
    X = torch.randn((batch * S, D), device=dev, generator=g).bfloat16()
    Wt = (torch.randn((3 * Hh * DH, D), device=dev, generator=g) * 0.02).bfloat16()
    for _ in range(warmup):
        eng.qkv_project(X, Wt, batch, S, Hh, absmax=True)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    ev[0].record()
    for _ in range(steps):
        Q, K, V, ka, va = eng.qkv_project(X, Wt, batch, S, Hh, absmax=True)
    ev[1].record()
    eng.synchronize()
    ms = ev[0].elapsed_time(ev[1]) / steps
    flops = 2.0 * batch * S * D * 3 * Hh * DH
    # spot check against an fp64 product of the same BF16 operands
    rows = torch.tensor([0, 1, S - 1, batch * S - 1], device=dev)
    want = (X[rows].double() @ Wt[Hh * DH:Hh * DH + DH].double().t()).float()          # K of head 0
    got = torch.stack([K[int(r) // S, 0, int(r) % S].float() for r in rows])
    peaks = measured_peaks()
    return {"workload": f"qkv_projection_m{batch * S}_n{3 * Hh * DH}_k{D}_bf16", "ms_per_step": ms,
            "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "bound": "tensor", "peak": peaks["tensor"],
            "peak_kind": peaks["kind"] + " burst", "frac": flops / (ms * 1e-3) / 1e12 / peaks["tensor"],
            "max_abs_err_vs_fp64_product": float((got - want).abs().max())}


def measure_backward(eng, dev, steps, warmup, Bq=4) -> dict:
    """Attention backward at the prefill configuration's shape (B 4, H 16, S 4096, DH 64, fp32, causal with the
    Navier-Stokes prologue): dQ, dK, dV for a given dO.  Flops counted as the five products of the chain over the
    causal half (2.5 x the forward's); checked against the fp64 backward oracle on one short head first."""
    import numpy as np
    import torch
    import oracle as O
    from logos_b200 import lib as L
    p = L.Params.make(0.125, True, 0, 0, ETA, NU, 1.0, L.DIFFUSE_CAUSAL)
    g = torch.Generator(device=dev).manual_seed(91)
    small = [torch.randn((1, 1, 384, DH), device=dev, generator=g) for _ in range(4)]
    got = eng.attention_bwd(*small, p)
    want = O.attention_bwd(*(t.cpu().numpy() for t in small), O.attn_params(0.125, True, 0, 0, ETA, NU, 1.0, 1))
    err = max(float(np.abs(a.cpu().numpy() - b).max()) for a, b in zip(got, want))
    S = 4096
    Q, K, V, dO = (torch.randn((Bq, H, S, DH), device=dev, generator=g) for _ in range(4))
    for _ in range(warmup):
        eng.attention_bwd(Q, K, V, dO, p)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    ev[0].record()
    for _ in range(steps):
        eng.attention_bwd(Q, K, V, dO, p)
    ev[1].record()
    eng.synchronize()
    ms = ev[0].elapsed_time(ev[1]) / steps
    flops = 2.5 * 4.0 * Bq * H * S * S * DH / 2
    out = {"workload": f"attention_bwd_b{Bq}_h{H}_s{S}_dh{DH}_f32", "ms_per_step": ms,
           "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s (causal-halved, 5 products)", "bound": "fp32 FMA pipe",
           "max_abs_err_vs_oracle": err,
           "note": "exact fp32 arithmetic on the FMA pipe (no tensor cores): a first path for a row outside the forward hot path"}
    # the same gradients on the tensor cores (BF16 operands), checked against the fp32 kernels on the same operands
    Q16, K16, V16, dO16 = (t.bfloat16() for t in (Q, K, V, dO))
    ref32 = eng.attention_bwd(Q16.float(), K16.float(), V16.float(), dO16.float(), p)
    got16 = eng.attention_bwd16(Q16, K16, V16, dO16, p)
    eng.synchronize()
    err16 = max(float((a - b).abs().max() / b.abs().max().clamp_min(1.0)) for a, b in zip(got16, ref32))
    del ref32, got16
    for _ in range(warmup):
        eng.attention_bwd16(Q16, K16, V16, dO16, p)
    ev[0].record()
    for _ in range(steps):
        eng.attention_bwd16(Q16, K16, V16, dO16, p)
    ev[1].record()
    eng.synchronize()
    ms16 = ev[0].elapsed_time(ev[1]) / steps
    peaks = measured_peaks()
    out["tensor_cores_bf16"] = {"workload": f"attention_bwd16_b{Bq}_h{H}_s{S}_dh{DH}_bf16", "ms_per_step": ms16,
                                "value": flops / (ms16 * 1e-3) / 1e12, "unit": "TFLOP/s (causal-halved, 5 products)",
                                "frac_of_bf16_peak": flops / (ms16 * 1e-3) / 1e12 / peaks["tensor"],
                                "max_err_vs_fp32_kernels_rel_to_largest_gradient": err16}
    # the reference's own chain for one head at a length its seq x seq buffers allow
    path = os.path.join(os.path.dirname(os.path.abspath(O.__file__)), "_ref", "liblogos_refbwd.so")
    if os.path.exists(path):
        import ctypes as C
        ref = C.CDLL(path)
        ref.refbwd_attention_head.argtypes = [C.c_void_p] * 7 + [C.c_int, C.c_int, C.c_float, C.c_float, C.c_void_p, C.c_int]
        Sr = 2048
        q, k, v, do = (t[0, 0, :Sr].contiguous() for t in (Q, K, V, dO))
        dq, dk, dv = (torch.empty_like(q) for _ in range(3))
        scratch = torch.empty(3 * Sr * Sr + 3 * Sr * DH, dtype=torch.float32, device=dev)
        vp = lambda t: C.c_void_p(t.data_ptr())
        call = lambda: ref.refbwd_attention_head(vp(q), vp(k), vp(v), vp(do), vp(dq), vp(dk), vp(dv), Sr, DH, ETA, NU,
                                                 vp(scratch), 1)
        torch.cuda.synchronize()
        call()
        torch.cuda.synchronize()
        ev[0].record()
        for _ in range(3):
            call()
        ev[1].record()
        torch.cuda.synchronize()
        ref_ms = ev[0].elapsed_time(ev[1]) / 3
        one = [t[:1, :1, :Sr].contiguous() for t in (Q, K, V, dO)]
        eng.attention_bwd(*one, p)
        ev[0].record()
        for _ in range(3):
            eng.attention_bwd(*one, p)
        ev[1].record()
        eng.synchronize()
        out["one_head_s2048"] = {"reference_backward_chain_ms": ref_ms, "engine_ms": ev[0].elapsed_time(ev[1]) / 3}
    return out


def reference_gpu_kernels(eng, dev) -> list:
    """One head of the prefill and of the window configuration through the reference's own CUDA path
    (ns_advect_kernel + ns_diffuse_kernel + cuda_flash_attention_fwd, compiled unmodified for sm_100a)
    and through the engine on the same fp32 inputs: the fp32 drop-in entry point (exact arithmetic,
    no Navier-Stokes terms: the reference applies those in separate kernels) and the BF16 tensor-core path."""
    import torch
    import oracle as O
    from logos_b200 import lib as L
    G = O.refgpu()
    if G is None:
        return [{"unavailable": "oracle/_ref/liblogos_refgpu.so was not built"}]
    out = []
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]

    def timed(fn, n):
        fn()
        torch.cuda.synchronize()
        ev[0].record()
        for _ in range(n):
            fn()
        ev[1].record()
        torch.cuda.synchronize()
        return ev[0].elapsed_time(ev[1]) / n

    for name, S, window, stride in (("one head of causal_prefill s4096", 4096, 0, 0),
                                    ("one head of shunyam_window64_stride16 s8192", 8192, 64, 16)):
        g = torch.Generator(device=dev).manual_seed(3000 + S)
        Q, K, V = (torch.randn((S, DH), device=dev, generator=g) for _ in range(3))
        Qa, Vs, Oref, Oours = (torch.empty_like(Q) for _ in range(4))
        ptr = lambda t: t.data_ptr()

        def ref_path():
            G.refgpu_ns_advect(ptr(Q), ptr(Qa), S, DH, ETA)
            G.refgpu_ns_diffuse(ptr(V), ptr(Vs), S, DH, NU)
            G.refgpu_flash_attention_fwd(ptr(Qa), ptr(K), ptr(Vs), ptr(Oref), S, DH, 0.125, 1, int(window > 0), window, stride)

        def ref_kernel_only():
            G.refgpu_flash_attention_fwd(ptr(Qa), ptr(K), ptr(Vs), ptr(Oref), S, DH, 0.125, 1, int(window > 0), window, stride)

        t_ref = timed(ref_path, 3)
        t_ref_k = timed(ref_kernel_only, 3)
        t_f32 = timed(lambda: eng.flash_attention_fwd_f32(Qa, K, Vs, 0.125, True, window > 0, window, stride), 5)
        o32 = eng.flash_attention_fwd_f32(Qa, K, Vs, 0.125, True, window > 0, window, stride)
        p = L.Params.make(0.125, True, window, stride, ETA, NU, 1.0, L.DIFFUSE_CAUSAL)
        Qb, Kb, Vb = (t.bfloat16()[None, None].contiguous() for t in (Q, K, V))
        Ob = torch.empty_like(Qb)
        t_tc = timed(lambda: eng.attention(Qb, Kb, Vb, p, out=Ob), 10)
        eng.synchronize()
        out.append({"case": name, "reference_ns_plus_flash_kernel_ms": t_ref, "reference_flash_kernel_ms": t_ref_k,
                    "engine_f32_drop_in_ms": t_f32, "engine_bf16_fused_ms": t_tc,
                    "max_abs_f32_drop_in_vs_reference_kernel": float((o32 - Oref).abs().max()),
                    "max_abs_bf16_fused_vs_reference_path": float((Ob[0, 0].float() - Oref).abs().max())})
    return out


# ---------------------------------------------------------------------------------------------

def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    from logos_b200 import lib as L
    from logos_b200.engine import Comm, Engine
    from logos_b200.sharding import ShardedDecoder, connect_comm, head_range

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # a rank that falls out must end the others with an error, not leave them waiting
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    eng = Engine(local_rank)
    lo, hi = head_range(H, rank, world)
    Hl = hi - lo

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # one exchange block per rank, large enough for the biggest gathered tensor of the run
    comm = None
    if world > 1:
        biggest = B * H * DH * 4
        if args.workload != "decode" or not args.no_secondary:
            biggest = max(biggest, 8 * H * 8192 * DH * 2, 32 * H * 2048 * DH * 2)
        comm = Comm(eng, rank, world, biggest)
        connect_comm(comm)

    def finish():
        torch.cuda.synchronize()
        if comm is not None:
            barrier()
            comm.close()
        eng.close()
        if world > 1:
            dist.destroy_process_group()

    if args.workload == "qkv":
        r = measure_projection(eng, dev, args.batch if args.batch != 64 else 32, args.steps, args.warmup)
        print(json.dumps({"metric": r["workload"], "value": r["value"], "unit": r["unit"], "n_gpus": 1, "steps": args.steps,
                          "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
                          "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": {"workload": r["workload"]},
                          "max_abs_err_vs_fp64_product": r["max_abs_err_vs_fp64_product"],
                          "roofline": {"bound": "tensor", "achieved": r["value"], "peak": r["peak"], "peak_kind": r["peak_kind"],
                                       "frac": r["frac"], "traffic": None}, "gpu_launches": args.steps}))
        finish()
        return

    if args.workload == "bwd":
        r = measure_backward(eng, dev, max(3, args.steps // 4), 3, Bq=args.batch if args.batch != 64 else 4)
        print(json.dumps({"metric": r["workload"], "value": r["value"], "unit": r["unit"], "n_gpus": 1, "higher_is_better": True,
                          "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": {"workload": r["workload"]},
                          "detail": r}))
        finish()
        return

    if args.workload == "mma":
        # what one tcgen05.mma of the attention kernels' shapes costs a CTA that does nothing else
        # (logos_selftest_umma, timing modes): 32 x (4 | 8 | 8) MMAs back to back, clock cycles on the SM
        import torch
        from logos_b200 import lib as L
        res = {}
        for mode, n, name in ((0, 4, "ss_m128_n128_k16"), (1, 8, "ss_m128_n64_k16_b_mn_major"), (3, 8, "ts_m128_n64_k16"),
                              (32, 4, "ss_m128_n128_k16_elected_lane"), (33, 8, "ss_m128_n64_k16_b_mn_major_elected_lane"),
                              (35, 8, "ts_m128_n64_k16_elected_lane")):
            qk = (mode & 15) == 0
            A = torch.zeros((128, 64 if qk else 128), device=dev, dtype=torch.bfloat16)
            Bm = torch.zeros((128, 64), device=dev, dtype=torch.bfloat16)
            D = torch.zeros((128, 128 if qk else 64), device=dev)
            runs = []
            for _ in range(7):
                eng._check(eng.lib.logos_selftest_umma(eng.h, 16 + mode, L.BF16, A.data_ptr(), Bm.data_ptr(), D.data_ptr()))
                eng.synchronize()
                runs.append(float(D[0, 0]))
            nominal = 128 * (128 if qk else 64) * 16 * 2 / 8192.0
            res[name] = {"cycles_per_mma": sorted(runs)[3] / (32 * n), "cycles_at_8192_flop_per_clock": nominal}
        if rank == 0:
            print(json.dumps({"metric": "tcgen05_mma_cycles", "value": res["ss_m128_n128_k16"]["cycles_per_mma"], "unit": "cycles",
                              "n_gpus": world, "higher_is_better": False, "vs_baseline": None, "dtype": "bf16",
                              "data": "synthetic", "config": {"workload": "tcgen05_mma_back_to_back"}, "detail": res}))
        finish()
        return

    if args.workload == "stack":
        r = measure_stack(eng, dev, world, rank, comm, barrier, max_over_ranks)
        if rank == 0:
            print(json.dumps({"metric": "stack_decode_tokens_per_s", "value": r["tokens_per_s_decode"], "unit": "tokens/s",
                              "n_gpus": world, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                              "dtype": "bf16 projections, int8 KV", "data": "synthetic", "config": {"workload": r["workload"]},
                              "detail": r}))
        finish()
        return

    if args.workload in ("prefill", "prefill8k", "window", "window_lm"):
        cfg = dict({"prefill": PREFILL, "prefill8k": PREFILL_8K, "window": WINDOW, "window_lm": WINDOW_LM}[args.workload])
        if args.batch != 64:   # profiling case: fewer sequences than the configuration
            cfg["B"] = args.batch
            cfg["name"] += f"_batch{args.batch}"
        r = measure_attention(eng, dev, world, rank, cfg, args.steps, args.warmup, barrier, max_over_ranks, comm)
        if rank == 0:
            print(json.dumps({"metric": cfg["name"], "value": r["value"], "unit": r["unit"], "n_gpus": world,
                              "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"],
                              "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
                              "data": "synthetic", "config": {"workload": cfg["name"]},
                              "max_abs_err_vs_oracle": r["max_abs_err_vs_oracle"],
                              "roofline": {"bound": r["bound"], "achieved": r["value"], "peak": r["peak"],
                                           "peak_kind": r["peak_kind"], "frac": r["frac"], "traffic": None},
                              "gpu_launches": args.steps}))
        finish()
        return

    # ---- caches: enough independent sets that a pass never finds its bytes in L2 ----
    per_set = 2 * B * Hl * S_MAX * DH
    n_sets = max(1, -(-(512 << 20) // per_set))
    g = torch.Generator(device=dev).manual_seed(1000 * 4 + rank)
    params = L.Params.make(1.0 / 8.0, True, 0, 0, ETA, NU, 1.0, L.DIFFUSE_CAUSAL)
    eng.reserve(eng.decode_workspace_bytes(B, Hl, S_MAX, DH))
    decoders = []
    for _ in range(n_sets):
        kc = torch.empty((B, Hl, S_MAX, DH), dtype=torch.int8, device=dev)
        vc = torch.empty_like(kc)
        ks = torch.empty((B, Hl), dtype=torch.float32, device=dev)
        vs = torch.empty_like(ks)
        for b0 in range(0, B, 8):  # quantize 8 sequences at a time to bound the fp32 staging
            for cache, sc in ((kc, ks), (vc, vs)):
                x = torch.randn((8, Hl, S_MAX, DH), device=dev, generator=g)
                x[torch.rand(x.shape, device=dev, generator=g) < 0.01] *= 8
                _, s = eng.nikhilam_compress(x, cache=cache[b0:b0 + 8])
                sc[b0:b0 + 8] = s
                del x
        decoders.append(ShardedDecoder(eng, kc, vc, ks, vs, params, rank, world, gather="peer", comm=comm))
    torch.cuda.synchronize()

    dblock = torch.randn((4, B, Hl, DH), device=dev, generator=g).half()     # q | q_prev | k_new | v_new
    q, qp, kn, vn = dblock[0], dblock[1], dblock[2], dblock[3]
    lens = torch.full((B,), S_MAX, dtype=torch.int32, device=dev)
    # the step's host tensors in one pinned block, one after the other (q | q_prev | k_new | v_new | len): the entry
    # point sends them as one copy
    n16 = 4 * B * Hl * DH * 2
    hbuf = torch.empty(n16 + B * 4, dtype=torch.uint8).pin_memory()
    hblock = hbuf[:n16].view(torch.float16).view(4, B, Hl, DH)
    hblock.copy_(dblock.cpu())
    hq, hqp, hkn, hvn = hblock[0], hblock[1], hblock[2], hblock[3]
    hlens = hbuf[n16:].view(torch.int32)
    hlens.copy_(lens.cpu())
    hout = torch.empty((B, H, DH), dtype=torch.float32).pin_memory()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]

    def timed_loop(fn) -> float:
        """`steps` calls of fn(i) between two events, REPEATS times; the median repeat, max over ranks."""
        for i in range(args.warmup):
            fn(i)
        per = []
        for _ in range(REPEATS):
            barrier()
            ev[0].record()
            for i in range(args.steps):
                fn(args.warmup + i)
            ev[1].record()
            barrier()
            per.append(ev[0].elapsed_time(ev[1]) / args.steps)
        return max_over_ranks(median(per))

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()

    # ---- eager launches (reported for comparison) ----
    eager_ms = timed_loop(lambda i: decoders[i % n_sets].step(q, qp, kn, vn, lens))

    # ---- the decode kernel alone and the whole step, each as one CUDA graph per cache set ----
    kernel_graphs = []
    if not args.no_graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        eng.use_stream(side)
        with torch.cuda.stream(side):
            for d in decoders:
                gph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gph, stream=side, capture_error_mode="thread_local"):
                    eng.decode_int8(q, qp, d.kc, d.vc, d.ks, d.vs, lens, params, out=d.out_local)
                kernel_graphs.append(gph)
        eng.use_stream(torch.cuda.current_stream())
        torch.cuda.current_stream().wait_stream(side)
        barrier()
        for d in decoders:
            d.capture(q, qp, kn, vn, lens)
            barrier()
        kern_ms = timed_loop(lambda i: kernel_graphs[i % n_sets].replay())
        step_ms = timed_loop(lambda i: decoders[i % n_sets].replay())
        launch = "one CUDA graph per step"
    else:
        kev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        for i in range(args.steps):
            d = decoders[i % n_sets]
            kev[i][0].record()
            eng.decode_int8(q, qp, d.kc, d.vc, d.ks, d.vs, lens, params, out=d.out_local)
            kev[i][1].record()
        torch.cuda.synchronize()
        kern_ms = max_over_ranks(sum(a.elapsed_time(b) for a, b in kev) / args.steps)
        step_ms, launch = eager_ms, "eager"
    clocks = sampler.stop() if rank == 0 else None

    # ---- host-buffer step: `e2e` ----
    if world == 1:
        e2e_fn = lambda i: decoders[i % n_sets].step_host(hq, hqp, hkn, hvn, hlens, hout)
        e2e_how = "logos_decode_step_int8_host: copies, append, decode, copy back, synchronise"
    elif not args.no_graph:
        def e2e_fn(i):
            dblock.copy_(hblock, non_blocking=True)
            lens.copy_(hlens, non_blocking=True)
            hout.copy_(decoders[i % n_sets].replay(), non_blocking=True)
            torch.cuda.current_stream().synchronize()
        e2e_how = "pinned-host copies in, the step's graph, copy of the gathered rows back, synchronise"
    else:
        e2e_fn = lambda i: decoders[i % n_sets].step_host(hq, hqp, hkn, hvn, hlens, hout)
        e2e_how = "copies in, eager step, copy back, synchronise"
    e2e_ms = timed_loop(e2e_fn)

    total_bytes = algorithmic_bytes(B, H, S_MAX, DH)
    kernel_bytes = algorithmic_bytes(B, Hl, S_MAX, DH)
    peaks = measured_peaks()
    line = {
        "metric": METRIC, "value": total_bytes / (step_ms * 1e-3) / 1e9, "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8 KV, fp16 Q, fp32 accumulate", "data": "synthetic",
        "config": workload_config(world),
        "timing": {"launch": launch, "repeats": REPEATS, "statistic": "median over repeats of the mean step, max over ranks",
                   "ms_per_step_eager": eager_ms, "ms_per_step_graph": step_ms if launch != "eager" else None,
                   "gather": "peer-memory stores from the decode kernel + wait/copy kernel" if world > 1 else "none",
                   "l2": (f"inputs larger than L2: {per_set >> 20} MiB of cache per GPU per pass, "
                          f"{n_sets} cache set(s) visited in rotation")},
        "e2e": {"value": total_bytes / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
                "h2d_bytes_per_step": 4 * B * Hl * DH * 2 + B * 4, "d2h_bytes_per_step": B * H * DH * 4,
                "ms_per_step": e2e_ms, "how": e2e_how},
        "gpu_launches": (2 if world == 1 else 3) * args.steps * REPEATS,
        "roofline": {"bound": "hbm", "kernel": "decode_dense_kernel",
                     "achieved": kernel_bytes / (kern_ms * 1e-3) / 1e9, "peak": peaks["hbm"], "peak_kind": peaks["kind"],
                     "unit": "GB/s", "frac": kernel_bytes / (kern_ms * 1e-3) / 1e9 / peaks["hbm"],
                     "kernel_ms": kern_ms, "traffic": DECODE_TRAFFIC_PER_PAIR * B * Hl,
                     "how": "the kernel alone, replayed as a graph over the same rotating caches, same loop and statistic as value"},
        "clocks": clocks,
    }
    for d in decoders:
        d.release()
    for gph in kernel_graphs:
        gph.reset()
    kernel_graphs.clear()
    if not args.no_secondary:
        # the other kernels of the path, device-resident, a few steps each
        decoders.clear()
        torch.cuda.empty_cache()
        line["secondary"] = [measure_attention(eng, dev, world, rank, cfg, max(3, args.steps // 4), 3, barrier,
                                               max_over_ranks, comm)
                             for cfg in (PREFILL, PREFILL_8K, WINDOW, WINDOW_LM)]
        torch.cuda.empty_cache()
        line["stack"] = measure_stack(eng, dev, world, rank, comm, barrier, max_over_ranks)
        if world == 1:
            line["secondary"].append(measure_projection(eng, dev, 32, 5, 3))
            line["secondary"].append(measure_backward(eng, dev, 3, 2))
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["baselines"] = {"reference_gpu_kernels_on_this_gpu": reference_gpu_kernels(eng, dev),
                             "configuration_1_reference_cpu_forward": configuration1_cpu_baseline()}
        line["cpu_baseline"] = cpu_port_baseline()
    if rank == 0:
        print(json.dumps(line))
    decoders.clear()
    finish()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU legs and the reference's GPU kernels")
    ap.add_argument("--no-secondary", action="store_true", help="skip the prefill / window side measurements")
    ap.add_argument("--no-graph", action="store_true", help="time eager launches only")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "prefill8k", "window", "window_lm", "stack", "qkv", "bwd", "mma"],
                    help="decode is the benchmark; the others time one attention kernel alone (profiling)")
    ap.add_argument("--batch", type=int, default=B,
                    help="sequences in the batch; anything but the default is a profiling case, not the benchmark")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.batch != B:
        globals()["B"] = args.batch
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
