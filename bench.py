#!/usr/bin/env python
"""Benchmark of the attention hot path: Nikhilam INT8-KV decode attention at 8K context.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (one "step" = one decode step over the whole batch): 64 sequences, 16 heads,
DH 64, 8191 cached tokens + the new token; K/V pre-quantization values ~ N(0,1) with 1 %
outliers x8, quantized with one scale per (sequence, head, K|V) tensor; Q in FP16; the new
token is quantized on append, then attention streams the INT8 cache.  Heads are sharded
over the GPUs (total work fixed: strong scaling) and the outputs are all-gathered.

Prints ONE JSON line.  `value` times the device-resident step with CUDA events; `e2e` is
the same step through the host-buffer entry point with the copies inside the timed region.
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
# DRAM traffic of decode_dense_kernel per (sequence, head) pair at ctx 8192, from the ncu capture
# summarised in profiles/decode_dense_kernel_b16_ctx8192.md: 268.55 MB read + 4.20 MB written (mean of
# two launches) over 256 pairs.  Pairs are independent, so a launch moves this times its number of pairs.
DECODE_TRAFFIC_PER_PAIR = (268.55e6 + 4.20e6) / 256
METRIC = "int8_kv_decode_attention_bandwidth_8k_ctx"
UNIT = "GB/s"


def algorithmic_bytes(b: int, h: int, s: int, dh: int) -> int:
    """INT8 K + V read once, plus scales, Q/q_prev, the output and the appended rows."""
    return 2 * b * h * s * dh + 2 * b * h * 4 + 2 * b * h * dh * 2 + b * h * dh * 4 + 2 * b * h * dh


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


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
                                       "-lms", "100", "-i", str(self.idx)], stdout=self.f, stderr=subprocess.DEVNULL)
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


def run_reference(args) -> None:
    """The reference's own CPU attention (include/Attention.hpp, compiled unmodified) doing what
    a decode step costs in the reference today: a full re-forward of every (sequence, head)
    over its whole context (cuda/train_gpu.cu:2037-2046), heads farmed over all host threads.
    Each step is a bounded sample: one pair per thread at the full 8192-token context."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import ctypes as C
    import numpy as np
    import oracle as O
    R = O.ref()
    base = {"impl": "reference", "metric": METRIC, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
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
              "navier_stokes_attention over the whole context, last row is the decode output")
    base.update({"value": gbs, "ms_per_step": dt * 1e3, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                 "data": "synthetic",
                 "config": {"workload": "int8_kv_decode_b64_h16_ctx8192_dh64", "batch": B, "heads": H,
                            "ctx": S_MAX, "dh": DH},
                 "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": threads, "kind": "reference", "sample": sample},
                 "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
    print(json.dumps(base))


PREFILL = {"name": "causal_prefill_b4_h16_s4096_dh64_bf16", "B": 4, "S": 4096, "window": 0, "outliers": False}
WINDOW = {"name": "shunyam_window64_b8_h16_s8192_dh64_bf16", "B": 8, "S": 8192, "window": 64, "stride": 0,
          "outliers": True}
# the reference's production setting: window 64 plus every 16th key as a landmark (cuda/train_gpu.cu:1172-1173)
WINDOW_LM = {"name": "shunyam_window64_stride16_b8_h16_s8192_dh64_bf16", "B": 8, "S": 8192, "window": 64,
             "stride": 16, "outliers": True}


def measured_peak_tflops():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops"]), "measured burst"
    except Exception:
        return 1590.0, "fallback"


def measure_attention(eng, dev, world, rank, cfg, steps, warmup, barrier, max_over_ranks) -> dict:
    """Device-resident prefill / window attention over this rank's heads (BF16 in, BF16 out,
    Navier-Stokes prologue fused: eta 0.1, causal diffusion nu 0.05), outputs all-gathered."""
    import torch
    from logos_b200 import lib as L
    from logos_b200.sharding import all_gather_heads, head_range
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
    p = L.Params.make(1.0 / 8.0, True, cfg["window"], cfg.get("stride", 0), ETA, NU, 1.0, L.DIFFUSE_CAUSAL)

    def step(i):
        Q, K, V = sets[i % 2]
        eng.attention(Q, K, V, p, out=O)
        if world > 1:
            all_gather_heads(O, world)

    for i in range(warmup):
        step(i)
    barrier()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    ev[0].record()
    for i in range(steps):
        step(warmup + i)
    ev[1].record()
    barrier()
    eng.synchronize()
    ms = max_over_ranks(ev[0].elapsed_time(ev[1]) / steps)
    out = {"workload": cfg["name"], "ms_per_step": ms, "n_gpus": world}
    if cfg["window"]:
        nbytes = 4 * Bc * H * S * DH * 2                       # Q, K, V read once, O written once
        peak, kind = measured_peak_gbs()
        out.update({"value": nbytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "bound": "hbm", "peak": peak,
                    "peak_kind": kind, "frac": nbytes / (ms * 1e-3) / 1e9 / (peak * world)})
    else:
        flops = 4.0 * Bc * H * S * S * DH / 2                  # causal-halved convention
        peak, kind = measured_peak_tflops()
        out.update({"value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s (causal-halved)", "bound": "tensor",
                    "peak": peak, "peak_kind": kind, "frac": flops / (ms * 1e-3) / 1e12 / (peak * world)})
    return out


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    from logos_b200 import lib as L
    from logos_b200.engine import Engine
    from logos_b200.sharding import ShardedDecoder, head_range

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

    if args.workload in ("prefill", "window", "window_lm"):
        cfg = dict({"prefill": PREFILL, "window": WINDOW, "window_lm": WINDOW_LM}[args.workload])
        if args.batch != 64:   # profiling case: fewer sequences than the configuration
            cfg["B"] = args.batch
            cfg["name"] += f"_batch{args.batch}"
        r = measure_attention(eng, dev, world, rank, cfg, args.steps, args.warmup, barrier, max_over_ranks)
        if rank == 0:
            print(json.dumps({"metric": cfg["name"], "value": r["value"], "unit": r["unit"], "n_gpus": world,
                              "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"],
                              "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
                              "data": "synthetic", "config": {"workload": cfg["name"]},
                              "roofline": {"bound": r["bound"], "achieved": r["value"], "peak": r["peak"],
                                           "peak_kind": r["peak_kind"], "frac": r["frac"], "traffic": None},
                              "gpu_launches": args.steps}))
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- caches: enough independent sets that a pass never finds its bytes in L2 ----
    per_set = 2 * B * Hl * S_MAX * DH
    n_sets = max(1, -(-(512 << 20) // per_set))
    g = torch.Generator(device=dev).manual_seed(1000 * 4 + rank)
    params = L.Params.make(1.0 / 8.0, True, 0, 0, ETA, NU, 1.0, L.DIFFUSE_CAUSAL)
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
        decoders.append(ShardedDecoder(eng, kc, vc, ks, vs, params, rank, world))
    torch.cuda.synchronize()

    def new_tokens():
        return [torch.randn((B, Hl, DH), device=dev, generator=g).half() for _ in range(4)]

    q, qp, kn, vn = new_tokens()
    lens = torch.full((B,), S_MAX, dtype=torch.int32, device=dev)
    hq, hqp, hkn, hvn = (t.cpu().pin_memory() for t in (q, qp, kn, vn))
    hlens = lens.cpu().pin_memory()
    hout = torch.empty((B, H, DH), dtype=torch.float32).pin_memory()

    # ---- device-resident step: `value` ----
    for i in range(args.warmup):
        decoders[i % n_sets].step(q, qp, kn, vn, lens)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    kev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    ev[0].record()
    for i in range(args.steps):
        d = decoders[(args.warmup + i) % n_sets]
        torch.sub(lens, 1, out=d.pos)
        eng.kv_append(kn, vn, d.kc, d.vc, d.ks, d.vs, d.pos)
        kev[i][0].record()
        eng.decode_int8(q, qp, d.kc, d.vc, d.ks, d.vs, lens, params, out=d.out_local)
        kev[i][1].record()
        if world > 1:
            from logos_b200.sharding import all_gather_heads
            all_gather_heads(d.out_local, world)
    ev[1].record()
    barrier()
    step_ms = max_over_ranks(ev[0].elapsed_time(ev[1]) / args.steps)
    kern_ms = max_over_ranks(sum(a.elapsed_time(b) for a, b in kev) / args.steps)

    # ---- the same step replayed as one CUDA graph launch per step ----
    # (the eager loop above stays: it carries the per-kernel events behind `roofline`)
    graph_ms = None
    # One GPU only for now: with two and four ranks the replayed step measured 120 / 90 us against 150 / 126 us
    # eager, but the eight-rank run of the same code did not finish within its time limit.
    if not args.no_graph and world == 1:
        for d in decoders:
            d.capture(q, qp, kn, vn, lens)
        for i in range(args.warmup):
            decoders[i % n_sets].replay()
        barrier()
        ev[0].record()
        for i in range(args.steps):
            decoders[(args.warmup + i) % n_sets].replay()
        ev[1].record()
        barrier()
        graph_ms = max_over_ranks(ev[0].elapsed_time(ev[1]) / args.steps)
    clocks = sampler.stop() if rank == 0 else None      # sampled over the eager and the replayed loop
    eager_ms = step_ms
    if graph_ms is not None:      # `value` is the replayed step whenever it was measured
        step_ms = graph_ms

    # ---- host-buffer step: `e2e` ----
    for i in range(args.warmup):
        decoders[i % n_sets].step_host(hq, hqp, hkn, hvn, hlens, hout)
    barrier()
    ev[0].record()
    for i in range(args.steps):
        decoders[(args.warmup + i) % n_sets].step_host(hq, hqp, hkn, hvn, hlens, hout)
    ev[1].record()
    barrier()
    e2e_ms = max_over_ranks(ev[0].elapsed_time(ev[1]) / args.steps)

    total_bytes = algorithmic_bytes(B, H, S_MAX, DH)
    kernel_bytes = algorithmic_bytes(B, Hl, S_MAX, DH)
    peak, peak_kind = measured_peak_gbs()
    line = {
        "metric": METRIC, "value": total_bytes / (step_ms * 1e-3) / 1e9, "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8 KV, fp16 Q, fp32 accumulate", "data": "synthetic",
        "config": {"workload": f"int8_kv_decode_b{B}_h16_ctx8192_dh64", "batch": B, "heads": H, "ctx": S_MAX, "dh": DH,
                   "ns_eta": ETA, "ns_nu": NU, "diffusion": "causal", "parallelism": f"heads/{world}",
                   "launch": ("one CUDA graph per step" if graph_ms is not None else "eager"),
                   "ms_per_step_eager": eager_ms, "ms_per_step_graph": graph_ms,
                   "l2": (f"inputs larger than L2: {per_set >> 20} MiB of cache per GPU per pass, "
                          f"{n_sets} cache set(s) visited in rotation")},
        "e2e": {"value": total_bytes / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
                "h2d_bytes_per_step": 4 * B * Hl * DH * 2 + B * 4, "d2h_bytes_per_step": B * H * DH * 4,
                "ms_per_step": e2e_ms},
        "gpu_launches": 2 * args.steps,
        "roofline": {"bound": "hbm", "kernel": "decode_dense_kernel",
                     "achieved": kernel_bytes / (kern_ms * 1e-3) / 1e9, "peak": peak, "peak_kind": peak_kind,
                     "unit": "GB/s", "frac": kernel_bytes / (kern_ms * 1e-3) / 1e9 / peak,
                     "kernel_ms": kern_ms, "traffic": DECODE_TRAFFIC_PER_PAIR * B * Hl},
        "clocks": clocks,
    }
    if not args.no_secondary:
        # the other two kernels of the path, device-resident, a few steps each
        del decoders
        torch.cuda.empty_cache()
        line["secondary"] = [measure_attention(eng, dev, world, rank, cfg, max(3, args.steps // 4), 3, barrier,
                                               max_over_ranks) for cfg in (PREFILL, WINDOW, WINDOW_LM)]
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_port_baseline()
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="skip the prefill / window side measurements")
    ap.add_argument("--no-graph", action="store_true", help="skip the CUDA-graph replay of the decode step")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "window", "window_lm"],
                    help="decode is the benchmark; prefill / window time the other kernels alone (profiling)")
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
