#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers N] [--impl ours|reference]

A step is one decode step of the whole batch.  The default run has the layer sizes of GPT-2 medium
(n_embd 1024, n_head 16, n_inner 4096, vocab 50257, 1024 positions; 24 layers) with seeded random
bfloat16 weights, a batch of 8 requests with 512-token prompts and a context of 1024: after the
prompts are in the cache, W untimed and K timed decode steps follow.  One JSON line is printed:

  value      decoded tokens per second, timed on the device (CUDA events around the K steps): the median of
             five trials of K steps, each on fresh requests (`trials_ms` lists them).  The steps run as the
             scheduler runs them: each is a CUDA graph (model and sampler), launched one ahead of the tokens (the
             next step takes them on the device from the step in flight, the host reads them one step behind)
  e2e        the same through the Python entry point (BatchGenerator): host token ids in, host
             token ids out, every step's inputs copied from pinned host memory and its tokens read back
             (bytes counted at the copies); median of three trials
  prefill    one step of 2 x 1024 prompt tokens: tokens/s, ms, flops / time / measured bf16 peak
  roofline   decode step: bytes it has to read (every weight once + the live requests' cache) / time,
             against the measured copy bandwidth
  points     decode tokens/s at batch 1 and 64, the same from 1000-token prompts, and the mixed workload
             (64 requests, prompts of 16..1024 tokens, 256-token portions beside decoding requests)
  kernels    the kernels a decode step and a prefill step spend their time in, each kind timed alone (a CUDA
             graph of that kernel for every layer, L2 flushed between replays): microseconds per launch, the
             bytes or flops it has to move, and the fraction of the measured peak

With --gpus N > 1 it prints one line and exits with 2: the engine runs on one GPU.
"""
import argparse
import json
import os
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MEDIUM = dict(model_type="gpt2", n_layer=24, n_embd=1024, n_head=16, n_inner=4096, vocab_size=50257,
              n_positions=1024, layer_norm_epsilon=1e-5, activation_function="gelu_new")
SIZES = {"medium": MEDIUM,
         "large": dict(MEDIUM, n_layer=36, n_embd=1280, n_head=20, n_inner=5120),
         "xl": dict(MEDIUM, n_layer=48, n_embd=1600, n_head=25, n_inner=6400)}
PAGE_SIZE = 16
PROMPT_LEN = 512
CONTEXT = 1024


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index=0, period=0.1):
        self.period, self.samples, self._stop = period, [], threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append((mhz, reasons))
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if self.nv is None or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        nv = self.nv
        mhz = sorted(s[0] for s in self.samples)
        bits = 0
        for _, r in self.samples:
            bits |= r
        names = []
        for attr, name in (("nvmlClocksThrottleReasonHwSlowdown", "hw_slowdown"),
                           ("nvmlClocksThrottleReasonHwThermalSlowdown", "hw_thermal_slowdown"),
                           ("nvmlClocksThrottleReasonSwThermalSlowdown", "sw_thermal_slowdown"),
                           ("nvmlClocksThrottleReasonSwPowerCap", "sw_power_cap"),
                           ("nvmlClocksThrottleReasonHwPowerBrakeSlowdown", "hw_power_brake")):
            if bits & getattr(nv, attr, 0):
                names.append(name)
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": nv.nvmlDeviceGetMaxClockInfo(self.h, nv.NVML_CLOCK_SM),
                "reasons": names, "samples": len(mhz)}


def model_bytes_and_flops(cfg, n_layer):
    D, I, V = cfg["n_embd"], cfg["n_inner"] or 4 * cfg["n_embd"], cfg["vocab_size"]
    per_layer = D * 3 * D + D * D + 2 * D * I               # matrix elements
    vec = 3 * D + D + I + D + 4 * D                          # biases and norm vectors (float32)
    weight_bytes = n_layer * (2 * per_layer + 4 * vec) + 2 * V * D + 4 * 2 * D
    kv_bytes_per_token = n_layer * 2 * D * 2
    linear_flops_per_token = 2 * n_layer * per_layer
    return weight_bytes, kv_bytes_per_token, linear_flops_per_token


def decode_loop(engine, sampler_cls, model, batch, prompt_len, steps, warmup, vocab, seed=0):
    """Prefill `batch` prompts, then `warmup` + `steps` decode steps; returns (ms per step, launches per step)."""
    import torch

    from mlx_lm_b200 import ops
    from mlx_lm_b200.engine import StepEntry
    from mlx_lm_b200.engine.scheduler import Request
    from mlx_lm_b200.sampling import GREEDY

    g = torch.Generator().manual_seed(seed)
    sample = sampler_cls(model.device, seed=seed)
    reqs = []
    for b in range(batch):
        toks = torch.randint(0, vocab, (prompt_len,), generator=g).tolist()
        engine.add_request(1000 + b)
        reqs.append(Request(1000 + b, toks, prompt_len, 10 ** 9, GREEDY))
    for i in range(0, batch, 4):    # prompts, four requests a step
        chunk = reqs[i:i + 4]
        logits = engine.step([StepEntry(r.uid, r.tokens, [prompt_len - 1]) for r in chunk])
        toks, _ = sample(logits, chunk)
        for r, t in zip(chunk, toks):
            r.tokens.append(t)

    def run_steps(k):
        """k decode steps as the scheduler runs them: each is model and sampler in one CUDA graph; the step after
        it is launched (its tokens handed over on the device) before the host waits for this one's tokens."""
        rows = list(range(len(reqs)))
        flying = engine.decode_launch([StepEntry(r.uid, r.tokens[-1:], [0]) for r in reqs], reqs, sample)
        for i in range(k):
            ahead = None
            if i + 1 < k:
                ahead = engine.decode_launch([StepEntry(r.uid, [0], [0]) for r in reqs], reqs, sample,
                                             source=(flying, rows))
            toks, _ = engine.decode_collect(flying)
            for r, t in zip(reqs, toks):
                r.tokens.append(t)
            flying = ahead

    run_steps(warmup)
    torch.cuda.synchronize()
    ops.launch_count = 0
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    run_steps(steps)
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    launches = ops.launch_count / steps
    mean_ctx = prompt_len + 1 + warmup + (steps - 1) / 2.0
    engine.check_status()
    for r in reqs:
        engine.finish(r.uid)
    return ms, launches, mean_ctx


def print_timeline(prof, n_kernels, title):
    """The last `n_kernels` kernels of a torch.profiler capture: their start, their end and the time from the end
    of the kernel before to their own end (`chain`: what the kernel adds to the step, since each waits for the one
    before).  Kernels start before their predecessor ends (programmatic dependent launch), so durations overlap
    and only `chain` adds up.  Times under a profiler are for shares, not for the record."""
    import collections

    import torch

    ev = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA
          and "Memcpy" not in e.name and "Memset" not in e.name]
    ev.sort(key=lambda e: e.time_range.start)
    step = ev[-int(n_kernels):]
    t0 = step[0].time_range.start
    rows, prev_end = [], t0
    for e in step:
        rows.append((e.name.replace("void ", "")[:60], e.time_range.start - t0, e.time_range.end - t0,
                     e.time_range.end - prev_end))
        prev_end = e.time_range.end
    print(f"{title}: {len(rows)} kernels, {rows[-1][2]:.1f} us from the first start to the last end")
    mid = len(rows) // 2
    for name, a, b, chain in rows[mid:mid + 15]:
        print(f"  {name:60s} start {a:8.1f}  end {b:8.1f}  chain {chain:5.1f}")
    agg = collections.OrderedDict()
    for name, a, b, chain in rows:
        n, c, d = agg.get(name, (0, 0.0, 0.0))
        agg[name] = (n + 1, c + chain, d + b - a)
    for name, (n, c, d) in agg.items():
        print(f"  {n:3d} x {name:60s} chain {c / n:6.2f} us each ({100 * c / rows[-1][2]:4.1f} % of the step), "
              f"start to end {d / n:6.2f}")


def decode_timeline(engine, sampler_cls, model, batch, vocab):
    """Where a decode step's time goes, kernel by kernel: a few steps under torch.profiler (CUPTI)."""
    import torch
    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        _, launches, _ = decode_loop(engine, sampler_cls, model, batch, PROMPT_LEN, 3, 8, vocab)
        torch.cuda.synchronize()
    print_timeline(prof, launches, f"one decode step, batch {batch}")


def prefill_timeline(engine, n_prompts, vocab):
    """The same for one step of `n_prompts` whole prompts of 1024 tokens."""
    import torch
    from torch.profiler import ProfilerActivity, profile

    from mlx_lm_b200 import ops
    from mlx_lm_b200.engine import StepEntry

    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, vocab, (1024,), generator=g).tolist() for _ in range(n_prompts)]
    launches = 0
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for it in range(3):
            for i in range(n_prompts):
                engine.add_request(("pf", i))
            ops.launch_count = 0
            engine.step([StepEntry(("pf", i), prompts[i], [1023]) for i in range(n_prompts)])
            launches = ops.launch_count
            torch.cuda.synchronize()
            for i in range(n_prompts):
                engine.finish(("pf", i))
    print_timeline(prof, launches, f"one prefill step, {n_prompts} x 1024 tokens")


def mixed_workload(model, engine, vocab, args, n_requests=64, new_tokens=128, seed=3):
    """Continuous batching: 64 requests, prompt lengths uniform in [16, 1024], up to 128 new tokens each (fewer
    where the 1024 positions end first), portions of 256 tokens beside decoding requests, everything through the
    scheduler; wall-clock tokens per second."""
    import torch

    from mlx_lm_b200.generate import BatchGenerator

    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(16, 1025, (n_requests,), generator=g).tolist()
    prompts = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]
    new = [max(1, min(new_tokens, 1024 + 1 - n)) for n in lens]     # the last new token needs no position

    def run():
        gen = BatchGenerator(model, max_tokens=new_tokens, engine=engine, completion_batch_size=64,
                             prefill_batch_size=8, prefill_step_size=256, max_tokens_per_step=2048, seed=0)
        gen.insert(prompts, new)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        n_out = 0
        while gen.scheduler.has_work():
            n_out += len(gen.next()[1])
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        st = gen.scheduler.stats
        return dt, n_out, st

    run()                                   # warm-up: graphs, launch plans, workspaces
    before = engine.n_replayed
    dt, n_out, st = run()
    engine.check_status()
    return {"only": "mixed", "size": args.size, "requests": n_requests, "prompt_tokens": sum(lens),
            "generated_tokens": n_out, "seconds": round(dt, 4), "steps": st.steps,
            "prompt_tokens_per_s": round(sum(lens) / dt, 1), "generated_tokens_per_s": round(n_out / dt, 1),
            "tokens_per_s": round((sum(lens) + n_out) / dt, 1), "preemptions": st.preemptions,
            "replayed_steps": engine.n_replayed - before}


def reference_arm():
    """The reference is mlx-lm, installed without its dependencies under baseline/_ref.  It runs on MLX, for
    which this machine has no wheel: try the imports a run would need and report what this box answers."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "mlx_lm")):
        return {"impl": "reference", "unavailable": f"mlx-lm is not installed under baseline/_ref ({ref} has no mlx_lm)"}
    sys.path.insert(0, ref)
    tried = []
    for name in ("mlx.core", "mlx_lm"):
        try:
            __import__(name)
            tried.append(f"import {name}: ok")
        except BaseException as e:      # whatever this box raises is the answer
            tried.append(f"import {name}: {type(e).__name__}: {e}")
            return {"impl": "reference", "unavailable": "; ".join(tried) + " (mlx-lm runs on MLX, which has no "
                    "wheel for this machine and cannot be fetched: no network)"}
    return {"impl": "reference", "unavailable": "; ".join(tried) + "; mlx imports here, but the reference arm was never "
            "built because it never did before"}


def flush_l2(buf):
    buf.zero_()


def kernel_table(calls, pk, mode, attention_bytes=0.0, attention_flops=0.0, reps=5):
    """Each kind of kernel of a recorded step, timed alone: the launches of a kind (one per layer) are captured
    into a CUDA graph with their recorded arguments and replayed `reps` times with an L2 flush before each; the
    result is microseconds per launch, what the launch has to move (from the labels the parts gave, attention
    from the caller) and the fraction of the measured peak: HBM bytes for a decode step, bf16 flops for prefill."""
    import collections
    import re

    import torch

    groups = collections.OrderedDict()
    for c in calls:
        lab = c[4] or ("?", 0.0, 0.0)
        kind = re.sub(r"\.\d+\.", ".", lab[0])
        kind = re.sub(r"^h\.", "", kind)
        groups.setdefault(kind, []).append(c)
    side = torch.cuda.Stream()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def time_graph(launches):
        """Median microseconds of a graph of these launches, L2 flushed before every replay."""
        graph = torch.cuda.CUDAGraph()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for f, lib, fname, args, _ in launches:            # once eagerly
                f(*args[:-1], side.cuda_stream)
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            handle = torch.cuda.current_stream().cuda_stream
            for f, lib, fname, args, _ in launches:
                f(*args[:-1], handle)
        times = []
        for _ in range(reps + 1):
            flush_l2(flush)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            graph.replay()
            e.record()
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e) * 1e3)
        return sorted(times[1:])[len(times[1:]) // 2]

    # A kind with a launch or two per step (embedding, final norm, output head, sampler) is timed behind the
    # launches of the kind with the most launches, as the difference to those alone: a graph of one kernel would
    # mostly measure the graph's own launch.
    lead_kind = max(groups, key=lambda k: len(groups[k]))
    lead = groups[lead_kind] if len(groups[lead_kind]) >= 8 else []
    lead_us = time_graph(lead) if lead else 0.0
    out = collections.OrderedDict()
    for kind, group in groups.items():
        if len(group) >= 8 or not lead:
            us = (lead_us if kind == lead_kind else time_graph(group)) / len(group)
        else:
            us = max(time_graph(lead + group) - lead_us, 0.0) / len(group)
        flops = sum(c[4][1] for c in group if c[4]) / len(group)
        nbytes = sum(c[4][2] for c in group if c[4]) / len(group)
        if kind.endswith("attention"):
            flops, nbytes = attention_flops, attention_bytes
        rec = {"n": len(group), "us": round(us, 2)}
        if us <= 0.0:          # lost in the noise of the launches it was timed behind (a model of very few layers)
            out[kind] = rec
            continue
        if nbytes:
            rec["gbs"] = round(nbytes / us / 1e3, 1)
        if flops:
            rec["tflops"] = round(flops / us / 1e6, 1)
        if mode == "decode" and nbytes:
            rec["frac"] = round(nbytes / (us * 1e-6) / 1e9 / pk["hbm_gbs"], 3)
        elif mode == "prefill" and flops:
            rec["frac"] = round(flops / (us * 1e-6) / 1e12 / pk["bf16_tflops"], 3)
        out[kind] = rec
    return out


def decode_kernels(engine, batch, mean_ctx, cfg, pk):
    """The kernel table of the decode step at `batch` (the graph of that bucket must have run)."""
    import torch

    from mlx_lm_b200 import ops
    graph = engine._graphs[(next(b for b in engine.GRAPH_BUCKETS if b >= batch), False)]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        ops.start_recording()
        try:
            graph._launch()
        finally:
            calls = ops.stop_recording()
    side.synchronize()
    kv_bytes = batch * mean_ctx * 2 * cfg["n_embd"] * 2
    return kernel_table(calls, pk, "decode", attention_bytes=kv_bytes, attention_flops=2 * kv_bytes)


def matmul_yardstick(cfg, rows=(2048, 16384), variants=("library", "ours", "ours, single CTAs", "ours, pairs of CTAs"),
                     n_weights=8, reps=6):
    """torch.matmul (cuBLAS) and the engine's own tcgen05 linear kernel (as its launcher picks tiles, then forced to
    single CTAs and to pairs) on the model's four linear shapes, timed like the kinds of `kernel_table`: eight weight
    matrices a shape in one CUDA graph, L2 flushed before every replay, CUDA events; no bias, no epilogue.  The
    library is a yardstick only: it is nowhere on the engine's path."""
    import torch
    from mlx_lm_b200 import ops

    D, I = cfg["n_embd"], cfg["n_inner"] or 4 * cfg["n_embd"]
    shapes = {"c_attn": (3 * D, D), "attn.c_proj": (D, D), "mlp.c_fc": (I, D), "mlp.c_proj": (D, I)}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    side = torch.cuda.Stream()
    for M in rows:
        for name, (N, K) in shapes.items():
            x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
            ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) for _ in range(n_weights)]
            out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
            line = []
            for variant in variants:
                os.environ.pop("MLXB_TC_PAIR", None)
                if variant.endswith("single CTAs"):
                    os.environ["MLXB_TC_PAIR"] = "0"
                elif variant.endswith("pairs of CTAs"):
                    os.environ["MLXB_TC_PAIR"] = "1"

                def product(w):
                    if variant == "library":
                        torch.matmul(x, w.t(), out=out)
                    else:
                        ops.linear_tensor_cores(x, w, None, out, status, side.cuda_stream)

                with torch.cuda.stream(side):
                    for w in ws:
                        product(w)
                side.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    for w in ws:
                        product(w)
                times = []
                for _ in range(reps):
                    flush_l2(flush)
                    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    s.record()
                    graph.replay()
                    e.record()
                    torch.cuda.synchronize()
                    times.append(s.elapsed_time(e) * 1e3 / len(ws))
                us = sorted(times[1:])[(len(times) - 1) // 2]
                line.append(f"{variant} {us:.2f} us, {2.0 * M * N * K / us / 1e6:.0f} TFLOP/s")
            os.environ.pop("MLXB_TC_PAIR", None)
            print(f"{M:5d} rows  {name:12s} {N} x {K}:  " + ";  ".join(line), flush=True)
    assert int(status.item()) == 0


def run_ours(args):
    import torch

    from mlx_lm_b200 import ops
    from mlx_lm_b200.engine import Engine, StepEntry
    from mlx_lm_b200.generate import BatchGenerator
    from mlx_lm_b200.sampling.device import DeviceSampler
    from mlx_lm_b200.weights import load_model, write_random_model

    pk = peaks()
    cfg = dict(SIZES[args.size])
    n_layer_full = cfg["n_layer"]
    cfg["n_layer"] = args.layers or n_layer_full
    B, K, W = args.batch, args.steps, args.warmup
    if PROMPT_LEN + 1 + W + K > CONTEXT:
        raise SystemExit(f"--warmup {W} + --steps {K} decode steps after a {PROMPT_LEN}-token prompt exceed the "
                         f"context of {CONTEXT}")
    with tempfile.TemporaryDirectory() as d:
        write_random_model(d, cfg, seed=0)
        model, _ = load_model(d, dtype="bfloat16", device="cuda:0")
    vocab = cfg["vocab_size"]
    max_b = max(B, 64)
    engine = Engine(model, page_size=PAGE_SIZE, max_tokens=max_b * CONTEXT, max_requests=max_b)
    weight_bytes, kv_per_token, lin_flops = model_bytes_and_flops(cfg, cfg["n_layer"])

    if args.only == "mixed":
        print(json.dumps(mixed_workload(model, engine, vocab, args)))
        return
    if args.only == "yardstick":
        if args.prefill_prompts:     # a small case for a profiler: one row count, the engine's kernel only
            matmul_yardstick(cfg, rows=(1024 * args.prefill_prompts,), variants=("ours, single CTAs", "ours, pairs of CTAs"),
                             n_weights=1, reps=2)
        else:
            matmul_yardstick(cfg)
        return
    if args.only == "timeline":
        if args.prefill_prompts:
            prefill_timeline(engine, args.prefill_prompts, vocab)
        else:
            decode_timeline(engine, DeviceSampler, model, B, vocab)
        return
    if args.only == "decode":
        plen = args.prompt_len or PROMPT_LEN
        if plen + 1 + W + K > CONTEXT:
            raise SystemExit(f"--prompt-len {plen}: {W} + {K} decode steps after it exceed the context of {CONTEXT}")
        ms, launches, mean_ctx = decode_loop(engine, DeviceSampler, model, B, plen, K, W, vocab)
        step_bytes = weight_bytes + B * mean_ctx * kv_per_token
        print(json.dumps({"only": "decode", "batch": B, "prompt_len": plen, "mean_context": round(mean_ctx, 1),
                          "ms_per_step": round(ms, 4), "tokens_per_s": round(B / (ms / 1e3), 1),
                          "hbm_frac": round(step_bytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4),
                          "launches_per_step": launches}))
        return
    if args.only == "kernels":
        plen = args.prompt_len or PROMPT_LEN
        ms, launches, mean_ctx = decode_loop(engine, DeviceSampler, model, B, plen, 8, 3, vocab)
        table = decode_kernels(engine, B, mean_ctx, cfg, pk)
        print(f"decode step, batch {B}, context {mean_ctx:.0f}: {ms * 1e3:.1f} us, {launches:.0f} launches; "
              f"each kind alone:")
        for kind, r in table.items():
            print(f"  {kind:28s} x{r['n']:3d}  {r['us']:8.2f} us  {r.get('gbs', 0):8.1f} GB/s  "
                  f"{r.get('tflops', 0):7.1f} TFLOP/s  {r.get('frac', 0):6.3f} of the HBM peak")
        pf_ms, pf_table = prefill_step(engine, cfg, pk, vocab, args.prefill_prompts or 2, lin_flops, table=True)[1:]
        print(f"prefill step, {args.prefill_prompts or 2} x 1024 tokens: {pf_ms * 1e3:.1f} us; each kind alone:")
        for kind, r in pf_table.items():
            print(f"  {kind:28s} x{r['n']:3d}  {r['us']:8.2f} us  {r.get('gbs', 0):8.1f} GB/s  "
                  f"{r.get('tflops', 0):7.1f} TFLOP/s  {r.get('frac', 0):6.3f} of the bf16 peak")
        return

    # ---- prefill: 2 x 1024 tokens in one step (more prompts only with --only prefill --prefill-prompts N)
    n_pf = (args.prefill_prompts or 2) if args.only == "prefill" else 2
    if not 1 <= n_pf <= max_b:
        raise SystemExit(f"--prefill-prompts {n_pf}: 1 to {max_b}")
    prefill, pf_ms, pf_table = prefill_step(engine, cfg, pk, vocab, n_pf, lin_flops, table=not args.only)
    if args.only == "prefill":
        print(json.dumps({"only": "prefill", **prefill}))
        return

    # ---- decode, device-timed: five trials of K steps, each on fresh requests; the median counts
    trials = []
    with ClockSampler() as clocks:
        for t in range(5):
            ms, launches, mean_ctx = decode_loop(engine, DeviceSampler, model, B, PROMPT_LEN, K, W, vocab, seed=t)
            trials.append(ms)
    ms = sorted(trials)[len(trials) // 2]
    value = B / (ms / 1e3)
    step_bytes = weight_bytes + B * mean_ctx * kv_per_token
    achieved = step_bytes / (ms / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm_gbs"], 4)}
    kernels = {"decode": decode_kernels(engine, B, mean_ctx, cfg, pk), "prefill": pf_table}

    points = {}
    k_pts, w_pts = min(K, 64), max(3, min(W, 8))
    for b in (1, 64):
        pms = sorted(decode_loop(engine, DeviceSampler, model, b, PROMPT_LEN, k_pts, w_pts, vocab, seed=10 * b + t)[0]
                     for t in range(3))[1]
        points[f"decode_b{b}"] = round(b / (pms / 1e3), 1)
    for b in (1, 8, 64):       # the same from 1000-token prompts: the cache a step reads is twice as long
        pms = sorted(decode_loop(engine, DeviceSampler, model, b, 1000, 12, 8, vocab, seed=100 * b + t)[0]
                     for t in range(3))[1]
        points[f"decode_b{b}_prompt1000"] = round(b / (pms / 1e3), 1)
    mixed = mixed_workload(model, engine, vocab, args)
    points["mixed_64_requests_tokens_per_s"] = mixed["tokens_per_s"]
    points["mixed_generated_tokens_per_s"] = mixed["generated_tokens_per_s"]
    points["mixed_steps"] = mixed["steps"]
    points["mixed_replayed_steps"] = mixed["replayed_steps"]

    # ---- end to end through the Python entry point: host tokens in, host tokens out
    e2e_trials = []
    for t in range(3):
        g = torch.Generator().manual_seed(2 + t)
        host_prompts = [torch.randint(0, vocab, (PROMPT_LEN,), generator=g).tolist() for _ in range(B)]
        gen = BatchGenerator(model, max_tokens=W + K + 1, engine=engine, completion_batch_size=max(B, 8),
                             prefill_batch_size=max(B, 8), prefill_step_size=2048, max_tokens_per_step=4096, seed=0)
        gen.insert(host_prompts)
        n_out = 0
        while n_out < B * (1 + W):            # prompts and warm-up steps
            n_out += len(gen.next_generated())
        torch.cuda.synchronize()
        h2d0, d2h0 = engine.h2d_bytes, engine.d2h_bytes
        t0 = time.perf_counter()
        n_timed = 0
        for _ in range(K):
            n_timed += len(gen.next_generated())
        torch.cuda.synchronize()
        e2e_trials.append((n_timed / (time.perf_counter() - t0), (engine.h2d_bytes - h2d0) // K,
                           (engine.d2h_bytes - d2h0) // K))
        gen.close()
    e2e_trials.sort()
    e2e = {"value": round(e2e_trials[1][0], 1), "unit": "tokens/s", "h2d_bytes_per_step": int(e2e_trials[1][1]),
           "d2h_bytes_per_step": int(e2e_trials[1][2])}

    out = {
        "metric": f"decode tokens/s, GPT-2 {args.size}, batch {B}, 512-token prompts, context 1024",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights, uniform random prompt tokens",
        "config": {"model": f"gpt2-{args.size}", "n_layer": cfg["n_layer"], "n_layer_of_configuration": n_layer_full,
                   "n_embd": cfg["n_embd"], "n_head": cfg["n_head"], "n_inner": cfg["n_inner"],
                   "vocab_size": vocab, "n_positions": cfg["n_positions"], "global_batch": B,
                   "seq_len": CONTEXT, "prompt_len": PROMPT_LEN, "page_size": 16, "parallelism": "single_gpu",
                   "l2": "inputs larger than L2 (weights %.0f MB)" % (weight_bytes / 1e6),
                   "peaks": pk["source"], "prefill_peak": "bf16_tflops (burst)", "trials": len(trials)},
        "trials_ms": [round(t, 4) for t in trials],
        "clocks": clocks.summary(), "e2e": e2e, "gpu_launches": int(round(launches * K)),
        "prefill": prefill, "roofline": roofline, "points": points, "kernels": kernels, "impl": "ours",
    }
    print(json.dumps(out))


def prefill_step(engine, cfg, pk, vocab, n_pf, lin_flops, table=False):
    """One step of `n_pf` whole prompts of 1024 tokens, timed four times (the best of the last three counts)."""
    import torch

    from mlx_lm_b200.engine import StepEntry

    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, vocab, (1024,), generator=g).tolist() for _ in range(n_pf)]
    times = []
    for it in range(4):
        for i in range(n_pf):
            engine.add_request(("pf", i))
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        engine.step([StepEntry(("pf", i), prompts[i], [1023]) for i in range(n_pf)])
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
        for i in range(n_pf):
            engine.finish(("pf", i))
    pf_ms = min(times[1:])
    D, L = cfg["n_embd"], cfg["n_layer"]
    attn_layer = n_pf * 4 * D * (1024 * 1025 // 2)        # QK^T and PV over the causal half of every prompt
    pf_flops = n_pf * 1024 * lin_flops + L * attn_layer + n_pf * 2 * D * vocab
    prefill = {"value": round(n_pf * 1024 / (pf_ms / 1e3), 1), "tokens": n_pf * 1024, "ms": round(pf_ms, 4),
               "frac": round(pf_flops / (pf_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
    tab = None
    if table and engine.last_calls:
        tab = kernel_table(engine.last_calls, pk, "prefill", attention_flops=attn_layer,
                           attention_bytes=n_pf * 1024 * 4 * D * 2)
    return prefill, pf_ms, tab


def main():
    global PAGE_SIZE
    ap = argparse.ArgumentParser()
    ap.add_argument("--page-size", type=int, default=16, help="positions per page of the key/value cache")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration's 24 (0 = all)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only", default="", choices=["", "decode", "prefill", "mixed", "timeline", "kernels", "yardstick"],
                    help="run just this part and print its figures (decode / prefill: short runs for profiling; "
                         "mixed: 64 requests with prompts of 16..1024 tokens through the scheduler, 256-token portions "
                         "beside decoding requests; timeline: every kernel of one step with its start and end, "
                         "from torch.profiler; kernels: each kind of kernel of a decode and a prefill step timed "
                         "alone, with bytes, flops and the fraction of the measured peak; yardstick: torch.matmul on the "
                         "model's linear shapes, to hold the hand-written kernels against)")
    ap.add_argument("--prefill-prompts", type=int, default=0,
                    help="with --only prefill: 1024-token prompts in the one step (default and the contract's figure: "
                         "2); with --only timeline: the timeline of such a step instead of a decode step")
    ap.add_argument("--prompt-len", type=int, default=0,
                    help="with --only decode: prompt length before the timed steps (default 512, the contract's)")
    ap.add_argument("--size", default="medium", choices=sorted(SIZES), help="layer sizes: GPT-2 medium, large or XL")
    a = ap.parse_args()
    PAGE_SIZE = a.page_size
    if a.impl == "reference":
        print(json.dumps(reference_arm()))
        return 0
    if a.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not offered")
        return 2
    a.warmup = max(a.warmup, 3)
    run_ours(a)
    return 0


if __name__ == "__main__":
    sys.exit(main())
