#!/usr/bin/env python3
"""Benchmark of the quantized-matmul hot path on B200.

Headline line (one JSON object on stdout): Q4_K decode GEMV, weight 8192 x 3072,
batch 1 -- GB/s of algorithmic bytes (GGUF weight bytes + f32 x + f32 y), timed
on the device over a ring of weight copies larger than L2, with the roofline
fraction against the measured HBM copy peak, the end-to-end figure through the
host-buffer launch surface, and the CPU baseline (the oracle's restatement of
the reference's x86 decode path) timed on this host's cores.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--extras]

Under torchrun (N > 1) every rank runs the same per-GPU workload on its own GPU
(weak scaling: the ranks are the row shards of an N-times taller matrix; a
column-split projection needs no collective) and rank 0 prints the line.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ROWS, COLS, KIND_NAME, KIND = 8192, 3072, "q4_k", 12
RING = 40  # weight copies cycled through: 40 x 14.16 MB = 566 MB, 4.5x the 126 MB L2
ALGO_BYTES = ROWS * (COLS // 256) * 144 + COLS * 4 + ROWS * 4  # 14 200 832
WORKLOAD = f"C1: Q4_K decode GEMV, weight {ROWS}x{COLS}, batch 1"
# the same dictionary in both arms (ours and --impl reference), so that the two lines name one configuration
CONFIG = {"workload": WORKLOAD, "algorithmic_bytes_per_step": ALGO_BYTES,
          "l2": f"inputs larger than the cache between timed iterations: ring of weight copies ({RING} x 14.2 MB on the GPU, 8 x 14.2 MB on the host)"}


def load_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows, self.proc, self.idx = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                for n, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                pass
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def synth(seed_w=0x5EED0000, seed_x=0xAC7):
    """Seeded synthetic inputs of the workload: W ~ N(0, 0.02^2) quantized by the
    reference's Q4_K encoder (oracle restatement), x ~ N(0, 1)."""
    from oracle import frink_oracle as fo
    w = (np.random.default_rng(seed_w).standard_normal((ROWS, COLS), dtype=np.float32) * np.float32(0.02))
    x = np.random.default_rng(seed_x).standard_normal(COLS, dtype=np.float32)
    return fo.encode(KIND, w), x


def cpu_gemv_rate(raw, x, seconds, threads):
    """GB/s of the oracle's x86 decode path (AVX2 fused f32 dot, rows over threads)."""
    from oracle import frink_oracle as fo
    ring = [raw.copy() for _ in range(8)]  # 113 MB: past the host's last-level cache
    fo.matvec_f32(KIND, ring[0], ROWS, COLS, x, threads=threads, simd=True)
    n, t0 = 0, time.perf_counter()
    while time.perf_counter() - t0 < seconds:
        fo.matvec_f32(KIND, ring[n % len(ring)], ROWS, COLS, x, threads=threads, simd=True)
        n += 1
    dt = time.perf_counter() - t0
    return ALGO_BYTES * n / dt / 1e9, n, dt


def cpu_model():
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("model name"):
                return line.split(":", 1)[1].strip()
    except Exception:
        pass
    return "unknown"


def run_reference(args, rank, world):
    """The reference arm: the reference's CPU implementation of the path (oracle
    port; the reference is Rust and there is no Rust toolchain to build it with)
    on all host threads.  A step is one full C1 GEMV."""
    if rank != 0:
        return
    from oracle import frink_oracle as fo
    raw, x = synth()
    threads = fo.host_threads()
    ring = [raw.copy() for _ in range(8)]
    for i in range(args.warmup):
        fo.matvec_f32(KIND, ring[i % 8], ROWS, COLS, x, threads=threads, simd=True)
    t0 = time.perf_counter()
    for i in range(args.steps):
        fo.matvec_f32(KIND, ring[i % 8], ROWS, COLS, x, threads=threads, simd=True)
    dt = time.perf_counter() - t0
    v = ALGO_BYTES * args.steps / dt / 1e9
    print(json.dumps({
        "impl": "reference", "metric": "q4_k_gemv_gbs", "value": v, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32 (fused dequant dot)", "data": "synthetic",
        "config": CONFIG, "arm": "frink CPU decode path (AVX2 fused f32 dot), C++ restatement of the reference (Rust; no toolchain here)",
        "cpu_baseline": {"value": v, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": f"{args.steps} full GEMVs over 8 weight copies; {cpu_model()}"},
        "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def graph_of(n, launch):
    import torch
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(n):
            launch(i)
    return g


def timed_launches(steps, ring, launch, warmup):
    """Device time of exactly `steps` launches (CUDA graph replays of `ring`
    launches each, plus one graph with the remainder), CUDA events on the
    replaying stream."""
    import torch
    q, r = divmod(steps, ring)
    g_full = graph_of(ring, launch) if q else None
    g_rem = graph_of(r, launch) if r else None
    for _ in range(max(1, -(-warmup // ring))):
        (g_full or g_rem).replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(q):
        g_full.replay()
    if g_rem:
        g_rem.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1)


def timed_steps(steps, ring, launch, warmup, min_launches=2000):
    """The timed region of `steps` launches, repeated: a region of a few dozen launches is
    ~100 us, and one sample of it carries a graph launch's own latency and loses the overlap
    of neighbouring launches at both ends.  The same `steps`-launch region is therefore
    recorded R times back to back into one CUDA graph (R * steps >= min_launches launches over
    the ring of weight copies), timed between ONE pair of CUDA events; the time of one region
    is that total / R.  A second pass replays a graph of one region R times, each between its
    own events, for the spread.  Returns (ms per region, dict)."""
    import torch
    repeats = max(1, -(-min_launches // steps))
    g_all = graph_of(repeats * steps, launch)
    g_one = graph_of(steps, launch)
    for _ in range(2):
        g_all.replay()
    for _ in range(max(1, -(-warmup // max(steps, 1)))):
        g_one.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g_all.replay()
    e1.record()
    torch.cuda.synchronize()
    total = e0.elapsed_time(e1)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(repeats)]
    for a0, a1 in ev:
        a0.record()
        g_one.replay()
        a1.record()
    torch.cuda.synchronize()
    ms = sorted(a0.elapsed_time(a1) for a0, a1 in ev)
    return total / repeats, {"repeats": repeats, "us_per_step": total / repeats / steps * 1e3, "single_region_us_per_step_min": ms[0] / steps * 1e3,
                             "single_region_us_per_step_median": ms[len(ms) // 2] / steps * 1e3, "single_region_us_per_step_max": ms[-1] / steps * 1e3}


# DRAM bytes one launch of the bench kernel moves, from one ncu capture of this kernel and shape
# (14 230 272 read + 0 written; the algorithmic bytes are 14 200 832)
NCU_DRAM_BYTES_PER_LAUNCH = 14230272


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4000)
    ap.add_argument("--warmup", type=int, default=200)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--extras", action="store_true", help="(kept for old command lines: the table of other kinds, batches and shapes is part of the default line)")
    ap.add_argument("--no-extras", action="store_true", help="skip the table of other kinds, batches and shapes")
    ap.add_argument("--no-models", action="store_true", help="skip the whole-model pp512 / tg128 block")
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--no-gemm", action="store_true", help="skip the prefill GEMM sweep (M = 512 against the three projection shapes)")
    ap.add_argument("--model", default=None, choices=["llama3b", "qwen3moe", "gptoss", "tiny"],
                    help="whole-model pp512 / tg128 tokens per second (the Llama-3.2-3B and Qwen3-30B-A3B shapes) instead of the GEMV line")
    ap.add_argument("--layers", type=int, default=0, help="with --model: override the layer count")
    ap.add_argument("--profile-region", choices=["pp", "tg", "tg_batch8"], default=None,
                    help="with --model: bracket this timed region with cudaProfilerStart/Stop (for a profiler run with capture off at start)")
    ap.add_argument("--watchdog", type=int, default=0, help="seconds after which all thread stacks are printed and the process exits")
    ap.add_argument("--no-tp-graph", action="store_true", help="--model under torchrun: launch the decode step eagerly instead of replaying a CUDA graph with the collectives captured")
    ap.add_argument("--nccl-only", action="store_true", help="under torchrun: sum decode rows with NCCL instead of the peer-memory all-reduce")
    ap.add_argument("--case", default=None, help="kind:rows:cols:batch -- plain launches of one GEMV shape (for ncu captures)")
    args = ap.parse_args()
    if args.watchdog:
        import faulthandler
        faulthandler.dump_traceback_later(args.watchdog, exit=True)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        return run_reference(args, rank, world)

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: this benchmark has no CPU fallback"}))
        sys.exit(1)
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from frink_b200 import device, gpu, build
    build.build()

    if args.case:
        return single_case(args)
    if args.model:
        return model_bench(args, rank, world, local)

    raw, x = synth()
    raw_d = torch.from_numpy(raw).cuda()
    ws = [device.Weights(raw_d, KIND, ROWS, COLS) for _ in range(RING)]
    xd = torch.from_numpy(x).cuda()
    yd = torch.empty((1, ROWS), dtype=torch.float32, device="cuda")

    def launch(i):
        device.gemv(ws[i % RING], xd, out=yd)

    for i in range(max(3, min(args.warmup, RING))):
        launch(i)
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    device.counters(reset=True)
    barrier()
    if rank == 0:
        sampler.start()
    barrier()
    ms, spread = timed_steps(args.steps, RING, launch, args.warmup)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    launches = args.steps * spread["repeats"]  # one kernel of this library per step, in every repeat of the timed region
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    value = world * ALGO_BYTES * args.steps / (ms * 1e-3) / 1e9
    per_gpu = value / world

    # ---- end to end: the host-buffer launch surface frink-core binds, pinned
    # host buffers, x up and y down inside the timed region, weights resident
    x_pin = torch.from_numpy(x).pin_memory()
    raws = [raw.copy() for _ in range(RING)]
    nb = COLS // 256
    # five regions of e2e_steps calls each, every region closed by a synchronize and reduced to the slowest rank; the
    # median region is reported (a region is tens of milliseconds, so one host hiccup would otherwise decide the figure)
    e2e_steps = max(400, min(args.steps, 1000))
    for i in range(RING):
        y_host = gpu.launch_q4_k_matvec(raws[i], x_pin.numpy(), ROWS, nb * 144, nb)
    regions = []
    for _ in range(5):
        barrier()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            y_host = gpu.launch_q4_k_matvec(raws[i % RING], x_pin.numpy(), ROWS, nb * 144, nb)
        torch.cuda.synchronize()
        sec = time.perf_counter() - t0
        if world > 1:
            t = torch.tensor([sec], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            sec = float(t.item())
        regions.append(sec)
    e2e_s = float(np.median(regions))
    e2e = world * ALGO_BYTES * e2e_steps / e2e_s / 1e9

    # ---- partitioned figures: the whole models (tensor / expert parallel under torchrun) and the row-split
    # projection with its collective.  Every rank takes part; rank 0 keeps the results.
    models, tp_split = {}, None
    for w_ in ws:
        w_.release()
    ws.clear()
    torch.cuda.empty_cache()
    comm = None
    if world > 1 and not args.nccl_only:
        from frink_b200.comm import Comm
        comm = Comm(arena_bytes=1 << 30)
    if not args.no_models:
        for name in ("llama3b", "qwen3moe", "gptoss"):
            r_ = run_model(name, rank, world, comm=comm)
            if rank == 0:
                models[name] = r_
    if world > 1:
        tp_split = tp_row_split(rank, world, comm)

    if rank != 0:
        leave(world)
        return

    peak, which = load_peaks()
    from oracle import frink_oracle as fo
    threads = fo.host_threads()
    cpu_v, cpu_n, cpu_dt = cpu_gemv_rate(raw, x, args.cpu_seconds if world == 1 else 2.0, threads)
    # parity spot check of what was timed (not part of any timed region)
    want = fo.matmul_f64(KIND, raw, ROWS, COLS, fo.q8_1_round(x))[0]
    got = yd.cpu().numpy()[0]
    rel = float(np.linalg.norm(got - want) / np.linalg.norm(want))
    rel_e2e = float(np.linalg.norm(y_host - want) / np.linalg.norm(want))

    line = {
        "metric": "q4_k_gemv_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 x int4 dp4a, f32 accumulate", "data": "synthetic",
        "config": CONFIG,
        "timing": f"the {args.steps}-launch region recorded {spread['repeats']} times back to back into one CUDA graph, one pair of CUDA events around its "
                  "replay; value and ms_per_step are that total per region; timing_spread: one region per graph, every replay timed on its own", "timing_spread": spread,
        "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak,
                     "traffic": NCU_DRAM_BYTES_PER_LAUNCH, "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this kernel and shape",
                     "peak_source": f"{which} HBM copy bandwidth", "frac_of_8TBs_nominal": per_gpu / 8000.0},
        "cpu_baseline": {"value": cpu_v, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": f"{cpu_n} full C1 GEMVs in {cpu_dt:.1f} s, AVX2 fused f32 dot, rows over threads; {cpu_model()}"},
        "e2e": {"value": e2e, "unit": "GB/s", "h2d_bytes_per_step": COLS * 4, "d2h_bytes_per_step": ROWS * 4,
                "steps": e2e_steps, "regions": 5, "ms_per_step": e2e_s / e2e_steps * 1e3,
                "ms_per_step_regions": [r_ / e2e_steps * 1e3 for r_ in regions],
                "api": "gpu.launch_q4_k_matvec(host weights, host x) -> host y, weights resident"},
        "gpu_launches": launches, "clocks": clocks,
        "parity": {"rel_l2_device": rel, "rel_l2_e2e": rel_e2e, "bar": 1e-3},
    }
    if models:
        line["models"] = models
    if tp_split:
        line["tp_row_split"] = tp_split
    if world == 1 and not args.no_gemm:
        line["gemm"] = gemm_sweep()
    if world == 1 and not args.no_extras:
        line["extras"] = extras(peak)
    print(json.dumps(line))
    leave(world)


def single_case(args):
    """`--case [gemv:|gemm:|gemm8k:]kind:rows:cols:n`: `--steps` plain (un-graphed) launches of
    one shape over a ring of weight copies larger than L2 (n = batch for the GEMV,
    tokens for the GEMM; gemm8k = the Q8_K-activation GEMM); the command the ncu captures run."""
    import torch
    from frink_b200 import device
    from oracle import frink_oracle as fo
    parts = args.case.split(":")
    op = parts.pop(0) if parts[0] in ("gemv", "gemm", "gemm8k") else "gemv"
    name, rows, cols, n = parts
    kind, rows, cols, n = fo.KINDS[name], int(rows), int(cols), int(n)
    rng = np.random.default_rng(1)
    base_rows = min(rows, 1024)
    base = fo.encode(kind, (rng.standard_normal((base_rows, cols), dtype=np.float32) * np.float32(0.02)))
    raw = np.tile(base, -(-rows // base_rows))[: rows * fo.row_bytes(kind, cols)]
    raw_d = torch.from_numpy(raw).cuda()
    ring = max(2, int(400e6 // raw.size) + 1)
    ws = [device.Weights(raw_d, kind, rows, cols) for _ in range(ring)]
    xd = torch.from_numpy(rng.standard_normal((n, cols), dtype=np.float32)).cuda()
    yd = torch.empty((n, rows), dtype=torch.float32, device="cuda")
    run = {"gemm": lambda i: device.gemm(ws[i % ring], xd, out=yd), "gemm8k": lambda i: device.gemm_q8k(ws[i % ring], xd, out=yd),
           "gemv": lambda i: device.gemv(ws[i % ring], xd, out=yd)}[op]
    for i in range(args.warmup):
        run(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        run(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    nbytes = raw.size + n * cols * 4 + n * rows * 4
    print(json.dumps({"case": args.case, "steps": args.steps, "us_per_launch_incl_host": ms / args.steps * 1e3,
                      "algorithmic_bytes": nbytes, "flops": 2.0 * n * rows * cols, "ring": ring,
                      "device_error_word": device.device_error()}))


def use_more_bits(i, n):
    """Which layers the Q4_K_M recipe gives Q6_K for attn_v / ffn_down
    (crates/frink-cli/src/quantize/recipe.rs, llama.cpp's rule)."""
    return i < n // 8 or i >= 7 * n // 8 or (i - n // 8) % 3 == 2


def synth_model(name, n_layers=0):
    """Random-init weights of the named shape, quantized by the reference's encoders
    (oracle restatement).  To keep set-up short, two sets of matrix bytes are quantized per
    shape; every layer takes one of them with its rows in an order of its own (and every
    expert of a layer a rotation of its own), so no two layers or experts apply the same
    matrix -- reused matrices add up coherently over the depth and a deep stack then answers
    every token with the same one, one route through the experts.  The embedding is 4096
    distinct rows tiled to the vocabulary.  `layers` is a generator (a layer's host bytes
    exist only until they are uploaded)."""
    from frink_b200.decoder import DecoderConfig, LayerWeights
    from oracle import frink_oracle as fo
    Q4, Q6, Q8 = fo.Q4_K, fo.Q6_K, fo.Q8_0
    if name == "llama3b":
        cfg = DecoderConfig(n_layers=28, hidden=3072, n_heads=24, n_kv=8, head_dim=128, ffn=8192, vocab=128256, rope_theta=500000.0, eps=1e-5)
    elif name == "qwen3moe":
        cfg = DecoderConfig(n_layers=48, hidden=2048, n_heads=32, n_kv=4, head_dim=128, ffn=768, vocab=151936, rope_theta=1000000.0,
                            eps=1e-6, neox=True, qk_norm=True, n_experts=128, top_k=8, route_mode=1)
    elif name == "gptoss":
        # gpt-oss-20b: BF16 attention projections with biases and sinks, every other layer windowed (128), 32 MXFP4 experts
        # (top 4) with biases and the clamped SwiGLU, BF16 embedding and head
        cfg = DecoderConfig(n_layers=24, hidden=2880, n_heads=64, n_kv=8, head_dim=64, ffn=2880, vocab=201088, rope_theta=150000.0,
                            eps=1e-5, neox=True, n_experts=32, top_k=4, route_mode=1, oai=True, sliding_window=128, swa_period=2)
    else:
        cfg = DecoderConfig(n_layers=2, hidden=512, n_heads=4, n_kv=2, head_dim=128, ffn=1024, vocab=4096)
    if n_layers:
        cfg.n_layers = n_layers
    rng = np.random.default_rng(0x5EED0000)
    H, hd = cfg.hidden, cfg.head_dim
    cache = {}
    # Norm weights of random sign: layers reuse two sets of matrix bytes, and the same matrices applied over and over
    # would pull the residual stream onto their dominant direction (one token for ever, one route through the experts);
    # a different sign pattern on every layer's input channels makes the layers act like different matrices.
    norm = lambda n: ((1.0 + 0.1 * rng.standard_normal(n)) * rng.choice([-1.0, 1.0], n)).astype(np.float32)

    def enc(tag, kind, rows, cols, variant):
        key = (tag, kind, rows, cols, variant)
        if key not in cache:
            base_rows = min(rows, 2048)
            # 0.02 everywhere but in the routed model, whose expert FFNs are narrow (768): there attention's output -- the same
            # vector for every position once the positions share a component, so it adds up coherently over 48 layers --
            # would swamp what depends on the token, and the stream would repeat one token (one route) for ever
            std = {"wo": 0.0005, "eg": 0.04, "eu": 0.04, "ed": 0.04}.get(tag, 0.02) if cfg.n_experts else 0.02
            w = (rng.standard_normal((base_rows, cols), dtype=np.float32) * np.float32(std))
            raw = fo.encode(kind, w)
            cache[key] = np.tile(raw, -(-rows // base_rows))[: rows * fo.row_bytes(kind, cols)].copy()
        return cache[key]

    def shuffled(raw, kind, rows, cols, seed):
        """The matrix with its rows in another order (whole quantized rows move, no byte changes)."""
        rb = fo.row_bytes(kind, cols)
        return raw.reshape(rows, rb)[np.random.default_rng(seed).permutation(rows)].ravel()

    def make_layers():
        # a generator: a layer's host bytes are built when the decoder asks for them and dropped after the upload
        for i in range(cfg.n_layers):
            var = i % 2
            sh = lambda tag, kind, r, c, j: shuffled(enc(tag, kind, r, c, var), kind, r, c, 7919 * i + j)
            if cfg.oai:
                BF, MX, E = fo.BF16, fo.MXFP4, cfg.n_experts
                kd = {"wq": BF, "wk": BF, "wv": BF, "wo": BF, "experts": MX}
                vec = lambda n_, s_: (rng.standard_normal(n_) * s_).astype(np.float32)

                def exo(tag, r, c, j):
                    base = sh(tag, MX, r, c, j).reshape(r, fo.row_bytes(MX, c))
                    idx = (np.arange(r)[None, :] + (np.arange(E) * 37 % r)[:, None]) % r
                    return base[idx].ravel()
                yield LayerWeights(
                    attn_norm=norm(H), wq=sh("wq", BF, cfg.n_heads * hd, H, 0), wk=sh("wk", BF, cfg.n_kv * hd, H, 1),
                    wv=sh("wv", BF, cfg.n_kv * hd, H, 2), wo=sh("wo", BF, H, cfg.n_heads * hd, 3), ffn_norm=norm(H),
                    gate=exo("eg", cfg.ffn, H, 4), up=exo("eu", cfg.ffn, H, 5), down=exo("ed", H, cfg.ffn, 6),
                    router=(rng.standard_normal((E, H), dtype=np.float32) * np.float32(0.02)), sinks=vec(cfg.n_heads, 1.0),
                    bq=vec(cfg.n_heads * hd, 0.02), bk=vec(cfg.n_kv * hd, 0.02), bv=vec(cfg.n_kv * hd, 0.02), bo=vec(H, 0.02),
                    router_bias=vec(E, 0.1), gate_b=vec(E * cfg.ffn, 0.02).reshape(E, cfg.ffn), up_b=vec(E * cfg.ffn, 0.02).reshape(E, cfg.ffn),
                    down_b=vec(E * H, 0.02).reshape(E, H), kinds=kd)
                continue
            if cfg.n_experts:
                kd = {"wq": Q8, "wk": Q8, "wv": Q8, "wo": Q8, "experts": Q4}
                E = cfg.n_experts

                def ex(tag, r, c, j):   # expert e = the layer's matrix with its rows rotated by a step of its own
                    base = sh(tag, Q4, r, c, j).reshape(r, fo.row_bytes(Q4, c))
                    idx = (np.arange(r)[None, :] + (np.arange(E) * 37 % r)[:, None]) % r
                    return base[idx].ravel()
                yield LayerWeights(
                    attn_norm=norm(H), wq=sh("wq", Q8, cfg.n_heads * hd, H, 0), wk=sh("wk", Q8, cfg.n_kv * hd, H, 1),
                    wv=sh("wv", Q8, cfg.n_kv * hd, H, 2), wo=sh("wo", Q8, H, cfg.n_heads * hd, 3), ffn_norm=norm(H),
                    gate=ex("eg", cfg.ffn, H, 4), up=ex("eu", cfg.ffn, H, 5), down=ex("ed", H, cfg.ffn, 6),
                    router=(rng.standard_normal((E, H), dtype=np.float32) * np.float32(0.02)),
                    # per-head q / k norms leave q and k at unit RMS: with weights near 1 the scores q.k / sqrt(d) reach +-11 and the
                    # softmax picks single keys, whose values then swamp the residual stream whatever the token; 0.3 keeps it soft
                    q_norm=norm(hd) * np.float32(0.3), k_norm=norm(hd) * np.float32(0.3), kinds=kd)
            else:
                more = use_more_bits(i, cfg.n_layers)
                kd = {"wq": Q4, "wk": Q4, "wv": Q6 if more else Q4, "wo": Q4, "gate": Q4, "up": Q4, "down": Q6 if more else Q4}
                yield LayerWeights(
                    attn_norm=norm(H), wq=sh("wq", kd["wq"], cfg.n_heads * hd, H, 0), wk=sh("wk", kd["wk"], cfg.n_kv * hd, H, 1),
                    wv=sh("wv", kd["wv"], cfg.n_kv * hd, H, 2), wo=sh("wo", kd["wo"], H, cfg.n_heads * hd, 3), ffn_norm=norm(H),
                    gate=sh("gate", kd["gate"], cfg.ffn, H, 4), up=sh("up", kd["up"], cfg.ffn, H, 5),
                    down=sh("down", kd["down"], H, cfg.ffn, 6), kinds=kd)
    layers = make_layers()
    tok_kind = fo.BF16 if cfg.oai else Q6

    def vocab_matrix_bf16(std):
        base = rng.standard_normal((4096, H), dtype=np.float32) * np.float32(std)
        copies = -(-cfg.vocab // 4096)
        # every copy of the 4096 rows at a scale of its own, so that no two rows of the vocabulary are the same
        parts = [fo.encode(tok_kind, base * np.float32(1.0 + 0.004 * c)) for c in range(copies)]
        return np.concatenate(parts)[: cfg.vocab * fo.row_bytes(tok_kind, H)].copy()

    if cfg.oai:
        return cfg, layers, vocab_matrix_bf16(1.0), tok_kind, norm(H), vocab_matrix_bf16(0.02)

    def vocab_matrix(std):
        base = fo.encode(tok_kind, (rng.standard_normal((4096, H), dtype=np.float32) * np.float32(std)))
        m = np.tile(base, -(-cfg.vocab // 4096))[: cfg.vocab * fo.row_bytes(tok_kind, H)].copy()
        # every copy of the 4096 rows gets its own super-block scale (the f16 at the end of each 210-byte Q6_K block), so
        # no two rows of the vocabulary are the same and an argmax does not fall back on the lowest id of a tie
        blocks = m.reshape(-1, 210)
        per_copy = 4096 * (H // 256)
        d16 = blocks[:, 208:210].copy().view(np.float16).astype(np.float32).ravel()
        d16 *= 1.0 + 0.004 * (np.arange(d16.size) // per_copy).astype(np.float32)
        blocks[:, 208:210] = d16.astype(np.float16).view(np.uint8).reshape(-1, 2)
        return m
    # An output head of its own (with a tied head a random-init model answers every token with itself) and an embedding
    # of unit scale, so that the token just read stays visible in the residual stream beside what the 0.02-scale
    # layers add: the greedy stream then moves from token to token and the router sees a different row every step.
    return cfg, layers, vocab_matrix(1.0), tok_kind, norm(H), vocab_matrix(0.02)


# per decode token, GGUF weight bytes every GPU streams together (layers + output head), and prefill matmul FLOPs of 512 tokens
# (routed shapes: the bytes of the CHOSEN experts, the attention, the router and the head; one GPU only -- under expert
# parallelism the replicated part does not divide by the ranks)
MODEL_ROOFLINE = {"llama3b": {"bytes_per_token": 2010839040, "pp512_flops": 2.89e12},
                  "qwen3moe": {"bytes_per_token": 2287392768, "pp512_flops": 2.80e12, "one_gpu_only": True},
                  "gptoss": {"bytes_per_token": 3710177280, "pp512_flops": 3.10e12, "one_gpu_only": True}}


def run_model(name, rank, world, n_layers=0, tp_graph=True, comm=None, profile_region=None):
    """pp512 / tg128 of a random-init model of the named shape: prefill of 512 random
    token ids (GEMM path), then 128 greedy tokens with the decode step replayed from a
    CUDA graph.  Under torchrun, dense layers are tensor parallel (NCCL all-reduce after
    wo / down) and experts expert parallel (replicated attention, one NCCL all-reduce of
    the partial expert sums per layer).  Times are CUDA events, max over ranks; weights
    stay resident.  Returns the result as a dict (rank 0) or None."""
    import torch
    import torch.distributed as dist
    from frink_b200 import device
    from frink_b200.decoder import Decoder
    cfg, layers, tok, tok_kind, out_norm, head = synth_model(name, n_layers)
    # dense models: tensor parallel; routed models: attention replicated, experts spread over the ranks
    # (their few KV heads do not divide by 8)
    try:
        dec = Decoder(cfg, layers, tok, tok_kind, out_norm, output=head, output_kind=tok_kind, max_seq=1024, dense_parallel=cfg.n_experts == 0,
                      comm=comm, prefill_acts="q8_k")
    except (ValueError, MemoryError) as e:      # (a shape that does not split over the ranks; an all-reduce arena that is full: the same on every rank)
        if world > 1:
            dist.barrier()
        return {"model": name, "n_gpus": world, "unavailable": str(e)} if rank == 0 else None
    del layers
    S, G = (512, 128) if name != "tiny" else (64, 16)
    prompt = torch.from_numpy(np.random.default_rng(0x70C).integers(0, cfg.vocab, S).astype(np.int32)).cuda()

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, region=None):
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if region is not None and region == profile_region:
            torch.cuda.profiler.start()      # a profiler started with its capture off takes only this region
        e0.record()
        r = fn()
        e1.record()
        sync()
        if region is not None and region == profile_region:
            torch.cuda.profiler.stop()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, r

    pp = []
    for _ in range(1 + 3):       # one warm-up, three timed
        dec.reset()
        ms, first = timed(lambda: dec.prefill(prompt), "pp" if _ == 3 else None)
        pp.append(ms)
    pp_ms = float(np.median(pp[1:]))
    cur = first.clone()
    use_graph = world == 1 or tp_graph
    if use_graph:
        g, out = dec.capture_decode(cur)
        step = lambda: (dec.replay(), cur.copy_(out))
    else:
        step = lambda: cur.copy_(dec.decode_step(cur))
    for _ in range(3):
        step()
    dec.pos.fill_(S)
    dec._pos_host = S
    toks = []

    def run_decode():
        for _ in range(G):
            step()
            toks.append(cur.clone())
    tg_ms, _ = timed(run_decode, "tg")
    # ---- a decode batch of eight independent sequences (their own KV caches and positions), one token each per step
    b8 = None
    if use_graph and (world == 1 or comm is not None):
        del step, g, out
        dec._graph = dec._gout = None
        NB8 = 8
        dec.alloc_seqs(NB8)
        cur8 = torch.cat([dec.prefill_seq(s_, prompt) for s_ in range(NB8)])
        # the sequences start from different tokens so that their routes differ
        cur8 = ((cur8 + torch.arange(NB8, device="cuda", dtype=torch.int32) * 37) % cfg.vocab).to(torch.int32).contiguous()
        g8, out8 = dec.capture_decode_seqs(cur8)
        step8 = lambda: (dec.replay_seqs(), cur8.copy_(out8))
        for _ in range(3):
            step8()
        seen8 = []

        def run8():
            for _ in range(G):
                step8()
                seen8.append(cur8.clone())
        b8_ms, _ = timed(run8, "tg_batch8")
        b8 = {"sequences": NB8, "steps": G, "ms": b8_ms, "tok_s": NB8 * G / (b8_ms * 1e-3),
              "distinct_tokens": len({int(v) for t_ in seen8 for v in t_.tolist()})}
        sync()
        del step8, g8, out8
        dec._graph_seqs = None
        use_graph = False
    err = device.device_error()
    wbytes = sum(v.w.gguf_bytes for L in dec.layers for v in L.values() if hasattr(v, "w") and hasattr(v.w, "gguf_bytes"))
    res = {
        "model": name, "n_gpus": world, "layers": cfg.n_layers,
        "pp_tokens": S, "pp_ms": pp_ms, "pp_tok_s": S / (pp_ms * 1e-3), "tg_tokens": G, "tg_ms": tg_ms, "tg_tok_s": G / (tg_ms * 1e-3),
        "decode_graph": bool(world == 1 or tp_graph),
        "prefill_activations": ("BF16 projections: f32 (library f32 GEMM for prompt rows, this library's matvec for decode); MXFP4 experts: q8_1" if cfg.oai else
                                "Q4_K projections: Q8_K (frink's CPU rule, per 256); other kinds: q8_1 (per 32); decode: q8_1"), "tg_batch8": b8, "parallelism": ("tp%d" % world) if not cfg.n_experts else ("dense replicated, ep%d" % world),
        "collective": None if world == 1 else (
            ("all-reduce(sum, f32 [rows, hidden]) after wo and down" if not cfg.n_experts else
             "all-reduce(sum, f32 [rows, hidden]) of the partial expert sums, one per layer") +
            ("; decode: in the epilogue of the row-split matvec (dense) / this library's all-reduce kernel (expert sums): peer stores over NVLink, "
             "each value with its arrival count, rank-order sum; prefill: NCCL" if comm is not None
             else "; NCCL")),
        "dense_weight_bytes_per_rank": wbytes, "device_error_word": err, "data": "synthetic random-init, quantized by the reference's encoders",
        "tokens_head": [int(t.item()) for t in toks[:8]], "distinct_tokens": len({int(t.item()) for t in toks})}
    roof = MODEL_ROOFLINE.get(name)
    if roof and not n_layers and (world == 1 or not roof.get("one_gpu_only")):
        hbm, _ = load_peaks()
        res["tg_frac_of_hbm"] = roof["bytes_per_token"] / world / (tg_ms / G * 1e-3) / 1e9 / hbm
        res["pp_tflops"] = roof["pp512_flops"] / (pp_ms * 1e-3) / 1e12
    # a live CUDA graph that holds captured collectives keeps the communicator busy: drop it before anything else uses the group
    sync()
    if use_graph:
        del step, g, out
        dec._graph = dec._gout = None
    del dec
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    return res if rank == 0 else None


def model_bench(args, rank, world, local):
    comm = None
    if world > 1 and not args.nccl_only:
        from frink_b200.comm import Comm
        comm = Comm(arena_bytes=1 << 30)
    res = run_model(args.model, rank, world, args.layers, not args.no_tp_graph, comm, args.profile_region)
    if rank == 0:
        res["metric"] = "pp512_tg128_tok_s"
        print(json.dumps(res))
    leave(world)


def leave(world):
    """After captured collectives were replayed, destroy_process_group() may never return: leave without the teardown."""
    import torch
    if world > 1:
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)


def tp_row_split(rank, world, comm=None, steps=400):
    """The row-split (K-split) projection of a decode step with its collective: the 3072 x 8192 Q4_K `down` matrix cut
    into K ranges of 8192 / world columns, one per rank, each rank's partial product summed over the ranks -- by NCCL,
    and by this library's peer-memory all-reduce.  Timed as a graph of `steps` such pairs (matvec over a ring of weight
    copies, then the reduction), CUDA events, max over ranks."""
    import torch
    import torch.distributed as dist
    from frink_b200 import device, parallel
    from oracle import frink_oracle as fo
    rows, cols = 3072, 8192
    rng = np.random.default_rng(7)
    base = fo.encode(fo.Q4_K, (rng.standard_normal((512, cols), dtype=np.float32) * np.float32(0.02)))
    raw = np.tile(base, rows // 512)
    local_raw, cl = parallel.shard_cols(raw, fo.Q4_K, rows, cols, rank, world)
    raw_d = torch.from_numpy(local_raw).cuda()
    ring = max(2, int(300e6 // local_raw.size) + 1)
    ws = [device.Weights(raw_d, fo.Q4_K, rows, cl) for _ in range(ring)]
    x = torch.from_numpy(rng.standard_normal((1, cl), dtype=np.float32)).cuda()
    y = torch.empty((1, rows), dtype=torch.float32, device="cuda")
    nbytes = rows * fo.row_bytes(fo.Q4_K, cols) + cols * 4 + rows * 4
    out = {"shape": f"Q4_K {rows}x{cols} cut into {world} K ranges of {cl} columns"}
    ch = comm.channel(rows) if comm is not None else None
    arms = ["nccl"] + (["peer_memory_kernel", "peer_memory"] if comm is not None else [])
    for name in arms:
        def launch(i):
            if name == "peer_memory":         # one launch: the matvec sums over the ranks in its epilogue
                device.gemv_fused(ws[i % ring], x, out=y, allreduce=(comm, ch))
                return
            device.gemv(ws[i % ring], x, out=y)
            if name == "nccl":
                dist.all_reduce(y, op=dist.ReduceOp.SUM)
            else:
                comm.all_reduce(ch, y)
        for i in range(5):
            launch(i)
        torch.cuda.synchronize()
        dist.barrier()
        g = graph_of(steps, launch)
        g.replay()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        del g
        out[name] = {"us_per_step": ms / steps * 1e3, "GBs_all_ranks": nbytes / (ms / steps * 1e-3) / 1e9,
                     "collective": {"nccl": "nccl all_reduce(sum, f32 [3072]) after every matvec",
                                    "peer_memory_kernel": "this library's all-reduce kernel after every matvec: peer stores over NVLink, each value with its arrival "
                                                          "count, rank-order sum",
                                    "peer_memory": "the same exchange in the matvec's own epilogue: one launch a step"}[name] + "; captured in the graph"}
    for w in ws:
        w.release()
    return out


def int8_peak_tops():
    """Dense int8 tensor throughput of this GPU as cuBLASLt delivers it (8192^3,
    torch._int_mm), the measured denominator beside the nominal 4500 TOPS."""
    import torch
    try:
        a = torch.randint(-127, 127, (8192, 8192), dtype=torch.int8, device="cuda")
        b = torch.randint(-127, 127, (8192, 8192), dtype=torch.int8, device="cuda").t()
        for _ in range(3):
            torch._int_mm(a, b)
        torch.cuda.synchronize()
        best = 1e9
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._int_mm(a, b)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return 2 * 8192 ** 3 / (best * 1e-3) / 1e12
    except Exception:
        return None


def gemm_sweep(m=512, steps=100, cpu_seconds=0.4):
    """The quantized prefill GEMM sweep: M = 512 tokens against 3072x3072, 8192x3072, 3072x8192
    in Q4_K, Q6_K, Q8_0 (plus MXFP4 on the 2880-wide shapes).  TFLOPS = 2*M*N*K over the whole
    call (activation quantization + plan + MMA kernel), CUDA-graph replays over a ring of weight
    copies larger than L2.  Two activation rules: "q8_1" (fk_gemm: per-32 scales, the decode
    kernels' rule, all kinds) and "q8_k" (fk_gemm_q8k: frink's CPU rule, per-256 scales, Q4_K).
    Beside every cell the reference's CPU batched path (Q8_K / Q8_0 activation quantization +
    integer row dots, the oracle port, not the 8-row repacked kernels) on all host threads, timed
    on a bounded sample of the tokens."""
    import torch
    from frink_b200 import device
    from oracle import frink_oracle as fo
    rng = np.random.default_rng(2)
    peak = int8_peak_tops()
    threads = fo.host_threads()
    cells = []
    shapes = [(3072, 3072), (8192, 3072), (3072, 8192)]
    todo = [(k, r, c) for k in ("q4_k", "q6_k", "q8_0") for (r, c) in shapes] + [("mxfp4", 2880, 2880), ("mxfp4", 8192, 2880)]
    for name, rows, cols in todo:
        kind = fo.KINDS[name]
        base_rows = min(rows, 512)
        base = fo.encode(kind, (rng.standard_normal((base_rows, cols), dtype=np.float32) * np.float32(0.02)))
        raw = np.tile(base, -(-rows // base_rows))[: rows * fo.row_bytes(kind, cols)]
        raw_d = torch.from_numpy(raw).cuda()
        ring = max(2, int(300e6 // raw.size) + 1)
        ws = [device.Weights(raw_d, kind, rows, cols) for _ in range(ring)]
        x = rng.standard_normal((m, cols), dtype=np.float32)
        xd = torch.from_numpy(x).cuda()
        out = torch.empty((m, rows), dtype=torch.float32, device="cuda")
        # the CPU arm: 16 tokens at a time until cpu_seconds have passed
        n_tok, t0 = 0, time.perf_counter()
        while time.perf_counter() - t0 < cpu_seconds:
            fo.matmul_q8(kind, raw, rows, cols, x[(n_tok % m):(n_tok % m) + 16], threads=threads)
            n_tok += 16
        cpu_tf = 2.0 * n_tok * rows * cols / (time.perf_counter() - t0) / 1e12
        rules = [("q8_1", device.gemm)] + ([("q8_k", device.gemm_q8k)] if name == "q4_k" else [])
        for rule, fn in rules:
            def launch(i):
                fn(ws[i % ring], xd, out=out)
            for i in range(3):
                launch(i)
            torch.cuda.synchronize()
            ms = timed_launches(steps, ring, launch, 10)
            tf = 2.0 * m * rows * cols * steps / (ms * 1e-3) / 1e12
            cells.append({"kind": name, "rows": rows, "cols": cols, "m": m, "activations": rule, "us": ms / steps * 1e3, "tflops": tf,
                          "frac_of_measured_int8": tf / peak if peak else None, "frac_of_nominal_4500": tf / 4500.0,
                          "cpu_baseline": {"value": cpu_tf, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                           "sample": f"{n_tok} of the {m} tokens; frink CPU vec_dot, non-repacked"}})
        for w in ws:
            w.release()
    err = device.device_error()
    return {"cells": cells, "int8_peak_tops_measured": peak, "int8_peak_tops_nominal": 4500.0, "device_error_word": err,
            "note": "q8_1: exact per-32-run integers, one f32 rescale per K = 32 MMA bounds it; q8_k: sub-block scales folded into the "
                    "int8 operand (two MMAs per K step), one drain per 256 K"}


def extras(peak):
    """Other kinds, batch sizes and a matrix large enough to amortise the launch."""
    import torch
    from frink_b200 import device
    from oracle import frink_oracle as fo
    out = []
    rng = np.random.default_rng(1)
    cases = [("q4_k", 12, 8192, 3072, 1), ("q4_k", 12, 8192, 3072, 2), ("q4_k", 12, 8192, 3072, 4), ("q4_k", 12, 8192, 3072, 8),
             ("q6_k", 14, 8192, 3072, 8), ("q8_0", 8, 8192, 3072, 8), ("mxfp4", 39, 8192, 2880, 8), ("q6_k", 14, 8192, 3072, 1), ("q8_0", 8, 8192, 3072, 1),
             ("mxfp4", 39, 8192, 2880, 1), ("q4_k", 12, 3072, 8192, 1), ("q6_k", 14, 128256, 3072, 1), ("q4_k", 12, 65536, 8192, 1),
             ("q5_k", 13, 8192, 3072, 1), ("q5_k", 13, 65536, 8192, 1),
             # gpt-oss-20b's BF16 tensors: the merged q/k/v projection and the output head
             ("bf16", 30, 5120, 2880, 1), ("bf16", 30, 201088, 2880, 1)]
    for name, kind, rows, cols, batch in cases:
        small = rows * cols <= 8192 * 8192
        base = fo.encode(kind, (rng.standard_normal((min(rows, 1024), cols), dtype=np.float32) * np.float32(0.02)))
        raw = np.tile(base, -(-rows // min(rows, 1024)))[: rows * fo.row_bytes(kind, cols)]
        raw_d = torch.from_numpy(raw).cuda()
        ring = max(2, int(600e6 // raw.size) + 1) if small else 2
        ws = [device.Weights(raw_d, kind, rows, cols) for _ in range(ring)]
        xd = torch.from_numpy(rng.standard_normal((batch, cols), dtype=np.float32)).cuda()
        yd = torch.empty((batch, rows), dtype=torch.float32, device="cuda")
        steps = 1000 if small else 60

        def launch(i):
            device.gemv(ws[i % ring], xd, out=yd)
        for i in range(3):
            launch(i)
        ms = timed_launches(steps, ring, launch, 20)
        nbytes = raw.size + batch * cols * 4 + batch * rows * 4
        gbs = nbytes * steps / (ms * 1e-3) / 1e9
        out.append({"kind": name, "rows": rows, "cols": cols, "batch": batch, "us": ms / steps * 1e3, "GBs": gbs, "frac": gbs / peak})
        for w in ws:
            w.release()
    return out


if __name__ == "__main__":
    main()
