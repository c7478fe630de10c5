#!/usr/bin/env python3
"""Benchmark of the decode step, a 2,048-token prefill and a mixed step at the shapes of Qwen2.5-7B, 14B
and 32B with random bfloat16 weights, on one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--shape 7b|14b|32b|config.json] [--batch 8]
                    [--context N] [--layers L] [--repeats R] [--mixed D,P] [--output FILE]

With no flags it runs the 7B shape (28 layers, batch 8, 8,192 tokens of context).  A "step" is one decode
step of the whole batch.  It prints ONE JSON line:
  value      decoded tokens per second: the median of R repeats, each timed on the device with CUDA events
             over exactly K steps after W warm-up steps; every request holds `context` tokens in the cache at
             the end of a repeat and feeds its last sampled token back on the device (no host round trip);
             `repeat_ms_per_step` lists all repeats
  e2e        the same through the Python entry point (InferenceService.run_cycle): every step copies the
             step's token ids from pinned host memory and reads the sampled ids and the status word back
  prefill    one step of 2,048 prompt tokens of one request, the median of R timed steps, each after a pause
             of 0.2 s (a prompt is a burst, not a sustained load); frac = flops / time / bf16 peak
  roofline   bytes the decode step has to read (every weight once, the live requests' cache) / its time,
             against the measured copy bandwidth
  points     decode tokens per second at batch 1 and 64 (points_roofline_frac: their share of the copy
             bandwidth, counted as for roofline)
  mixed      with --mixed D,P: ONE Engine.step of D decoding requests at the context beside one P-token
             portion of a prompt that has (context - P) / 2 tokens in the cache: device_ms (CUDA events around
             the step), host_ms (the host's clock from the call of Engine.step to its return, i.e. packing and
             launching, nothing waited for), the shares of the copy bandwidth and of the bf16 peak, and frac =
             roofline_ms / device_ms, where roofline_ms adds what the step's phases need one after the other: the
             decoding requests' cache at the copy bandwidth, the products at the bf16 peak (or their weights at the
             copy bandwidth, if that is longer), the portion's attention at the bf16 peak
The pool of cache pages is sized from the device memory that is free once the weights are resident.  The cache
of the decoding requests is filled with random keys and values instead of running 64 prompts (data: synthetic);
timing does not depend on the values.  Between timed steps nothing is flushed: a step reads its weights (over
14 GB at 28 layers), far more than the 126 MB of L2.
--impl reference runs EmersonDowell/AIR's own CUDA executor, built from its unmodified sources (baseline/),
on the same shape, batch and context, and prints the same line with "impl": "reference".
For --gpus N > 1 it prints one line that says so and exits with 2: this engine runs on one GPU.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

_QWEN = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "vocab_size": 152064,
         "max_position_embeddings": 32768, "rope_theta": 1000000.0, "tie_word_embeddings": False,
         "sliding_window": 131072, "use_sliding_window": False, "hidden_act": "silu"}
SHAPES = {
    "7b": dict(_QWEN, num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4,
               intermediate_size=18944, rms_norm_eps=1e-6, max_window_layers=28),
    "14b": dict(_QWEN, num_hidden_layers=48, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8,
                intermediate_size=13824, rms_norm_eps=1e-5, max_window_layers=48),
    "32b": dict(_QWEN, num_hidden_layers=64, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8,
                intermediate_size=27648, rms_norm_eps=1e-5, max_window_layers=64),
}
CONTEXTS = {"7b": 8192, "14b": 8192, "32b": 4096}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                d = json.load(f)
            found = {"hbm_gbs": _figure(d, "hbm_gbs"), "bf16_tflops": _figure(d, "bf16_tflops"), "source": "measured"}
            try:
                found["bf16_tflops_sustained"] = _figure(d, "bf16_tflops_sustained")
            except (ValueError, KeyError, TypeError):
                pass
            return found
        except (ValueError, KeyError, TypeError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


def _figure(record, key):
    """A peak from the record: a number, or an object that holds it under 'value' (or the key's own name); the
    key may also lie one level down (under 'peaks', say)."""
    if key not in record:
        for inner in record.values():
            if isinstance(inner, dict) and key in inner:
                record = inner
                break
    v = record[key]
    if isinstance(v, dict):
        v = v["value"] if "value" in v else v[key]
    v = float(v)
    if not v > 0:
        raise ValueError(key)
    return v


class ClockSampler:
    """nvidia-smi in the background during the timed region (reading only)."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.proc, self.lines = None, []
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def randomize_cache(engine, torch):
    """Random keys and values in every page of every run (once: pages keep them when they change hands)."""
    g = torch.Generator(device=engine.rt.device)
    g.manual_seed(1234)
    seen = set()
    for run in range(len(engine.model.spec.order)):
        for view in engine.cache.views(run):
            kv = getattr(view, "kv", None)
            if kv is None:
                kv = getattr(view, "rows", None)
            if kv is not None and kv.data_ptr() not in seen:
                seen.add(kv.data_ptr())
                kv.normal_(0.0, 0.5, generator=g)


def open_requests(engine, requests, tokens):
    """Opens the requests with `tokens` tokens each (whatever lies in their pages)."""
    for r in requests:
        engine.cache.open(r)
        engine.cache.reserve([(r, tokens)])
        engine.cache.commit(r, tokens)


def release(engine, requests):
    for r in requests:
        if r in engine.cache.sequences:
            engine.finish(r)


def decode_device(engine, requests, context, steps, warmup, repeats, torch, Entry, LAST):
    """R repeats of K decode steps timed with CUDA events; tokens are fed back on the device.  Every repeat
    starts from the same length, so that its last step runs at `context` tokens."""
    times, clocks, launches = [], None, 0
    start_len = context - (steps + warmup + 2)
    for rep in range(repeats):
        open_requests(engine, requests, start_len)
        first = [Entry(r, [17 + i], [0]) for i, r in enumerate(requests)]
        engine.sample(engine.step(first))
        again = [Entry(r, [LAST], [0]) for r in requests]
        for _ in range(warmup):
            engine.sample(engine.step(again))
        torch.cuda.synchronize()
        launches0 = engine.kernel_launches()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sampler = ClockSampler() if rep == 0 else None
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            engine.sample(engine.step(again))
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end) / steps)
        if sampler is not None:
            clocks = sampler.stop()
            launches = engine.kernel_launches() - launches0
        release(engine, requests)
    return times, clocks, launches


def decode_timeline(engine, requests, context, torch, Entry, LAST):
    """Spans of the kernels of one decode step as they run inside the CUDA graph (from the moment a
    kernel has passed the wait on its predecessor to the moment the next one has), by kernel."""
    import collections
    from air_b200.csrc import ops
    open_requests(engine, requests, context - 8)
    engine.sample(engine.step([Entry(r, [17 + i], [0]) for i, r in enumerate(requests)]))
    again = [Entry(r, [LAST], [0]) for r in requests]
    buf = torch.zeros(1 + 2 * 16384, dtype=torch.int64, device=engine.rt.device)
    ops.set_trace(buf)
    for _ in range(3):
        engine.sample(engine.step(again))
    torch.cuda.synchronize()
    ops.set_trace(None)
    release(engine, requests)
    b = buf.cpu().tolist()
    events = sorted((b[2 + 2 * i], b[1 + 2 * i]) for i in range(min(b[0], 16384)) if b[1 + 2 * i] < 100)
    start = [i for i, e in enumerate(events) if e[1] == 1][-1]           # the last step's embedding
    step = events[start:]
    spans = collections.defaultdict(lambda: [0, 0.0])
    for (t0, k), (t1, _) in zip(step, step[1:]):
        spans[ops.TRACE_NAMES[k]][0] += 1
        spans[ops.TRACE_NAMES[k]][1] += (t1 - t0) / 1e3
    total = (step[-1][0] - step[0][0]) / 1e3
    print(f"decode step inside the graph: {total:.1f} us from embedding to sampling, {len(step)} kernels")
    for name, (n, us) in sorted(spans.items(), key=lambda x: -x[1][1]):
        print(f"  {name:18s} {n:4d} launches {us:9.1f} us  {100 * us / total:5.1f} %  {us / n:7.1f} us each")
    # one layer from the middle of the step, kernel by kernel (from one attention kernel to the next)
    names = [ops.TRACE_NAMES[k] for _, k in step]
    marks = [i for i in range(len(step) // 2, len(step) - 1) if names[i] == "decode_attention"]
    if len(marks) >= 2:
        i, j = marks[0], marks[1]
        print("  one layer (us): " + " | ".join(f"{names[q]} {(step[q + 1][0] - step[q][0]) / 1e3:.1f}"
                                               for q in range(i, j)))


def prefill_timeline(engine, prompt, torch, Entry):
    """Spans between the starts of this package's kernels in one prefill step.  A library product has
    no trace point: its time is part of the span of the kernel before it."""
    import collections
    from air_b200.csrc import ops
    buf = torch.zeros(1 + 2 * 16384, dtype=torch.int64, device=engine.rt.device)
    ops.set_trace(buf)
    engine.step([Entry("p", prompt, [len(prompt) - 1])])
    torch.cuda.synchronize()
    ops.set_trace(None)
    engine.finish("p")
    b = buf.cpu().tolist()
    events = sorted((b[2 + 2 * i], b[1 + 2 * i]) for i in range(min(b[0], 16384)) if b[1 + 2 * i] < 100)
    spans = collections.defaultdict(lambda: [0, 0.0])
    order = []
    for (t0, k), (t1, k1) in zip(events, events[1:]):
        key = f"{ops.TRACE_NAMES[k]} -> {ops.TRACE_NAMES[k1]}"
        if key not in spans:
            order.append(key)
        spans[key][0] += 1
        spans[key][1] += (t1 - t0) / 1e3
    total = (events[-1][0] - events[0][0]) / 1e3
    print(f"prefill step of {len(prompt)} tokens: {total:.1f} us from embedding to sampling, {len(events)} traced kernels")
    for key in order:
        n, us = spans[key]
        print(f"  {key:42s} {n:4d} times {us:9.1f} us  {100 * us / total:5.1f} %  {us / n:7.1f} us each")


def decode_e2e(engine, requests, context, steps, warmup, torch):
    """The same through InferenceService.run_cycle, host tokens in and out every step."""
    from air_b200.engine.service import InferenceService, SchedulerConfig
    from air_b200.sampling.sampler import GenerationConfig
    open_requests(engine, requests, context - (steps + warmup + 2))
    service = InferenceService(engine, SchedulerConfig(max_active_requests=max(len(requests), 1),
                                                       token_budget_per_cycle=max(len(requests), 1)))
    for i, r in enumerate(requests):
        service.restore(r, 23 + i, GenerationConfig(max_new_tokens=steps + warmup + 1, stop_on_eos=False))
    for _ in range(warmup):
        service.run_cycle()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        service.run_cycle()
    torch.cuda.synchronize()
    sec = time.perf_counter() - t0
    release(engine, requests)
    # per step: 4 ints per token of the decode graph's batch from pinned memory; sampled ids and the status word back
    sizes = [g.size for g in engine.graphs.values() if g.size >= len(requests)]
    h2d = 16 * (min(sizes) if sizes else len(requests))
    return sec / steps, h2d, 4 * (len(requests) + 1)


def mixed_step(engine, decoders, portion, context, repeats, torch, Entry):
    """One Engine.step that holds `decoders` single next tokens of requests with `context` tokens and one portion of
    `portion` prompt tokens of a request that has (context - portion) / 2 tokens in the cache."""
    requests = [f"m{i}" for i in range(decoders)]
    prior = max(0, (context - portion) // 2 // 64 * 64)
    vocab = engine.model.spec.vocab_size
    g = torch.Generator().manual_seed(11)
    tokens = torch.randint(0, vocab, (portion,), generator=g).tolist()
    device_ms, host_ms = [], []
    for rep in range(repeats + 2):                 # the first two are warm-up
        open_requests(engine, requests, context - 1)
        open_requests(engine, ["portion"], prior)
        entries = [Entry(r, [5 + i], [0]) for i, r in enumerate(requests)] + [Entry("portion", tokens, [])]
        # (the pages of requests that earlier steps brought to their lengths are in the device's tables already:
        # without this the timed step would send the thousands of entries that opening the requests here made)
        engine.cache.flush_tables()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        t0 = time.perf_counter()
        logits = engine.step(entries)
        engine.sample(logits)
        t1 = time.perf_counter()
        end.record()
        torch.cuda.synchronize()
        if rep >= 2:
            device_ms.append(start.elapsed_time(end))
            host_ms.append((t1 - t0) * 1e3)
        release(engine, requests + ["portion"])
    return statistics.median(device_ms), statistics.median(host_ms), prior


def kernel_prefill_attention(cfg):
    """The tcgen05 attention kernel alone at the shape's heads: launches replayed as a CUDA graph of ten (a launch
    from the host costs more than the kernel takes), timed with CUDA events, median of five replays.  First one
    block per SM with streams of 4 to 128 key tiles (what a block costs beside its key tiles), then whole prompts
    and portions on top of long prefixes, with whole streams per block and with the planner's cut (if it cuts)."""
    import math
    import statistics
    import numpy as np
    import torch
    from air_b200.csrc import ops
    from air_b200.parts.attention import plan_segments
    d = cfg.get("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])
    heads, kv_heads, P = cfg["num_attention_heads"], cfg["num_key_value_heads"], 64

    def case(H, K, prior, portion):
        """One request, or several (lists): `portion` new tokens each behind `prior` tokens."""
        priors, portions = (prior, portion) if isinstance(prior, (list, tuple)) else ([prior], [portion])
        most = max(-(-(a + b) // P) for a, b in zip(priors, portions))
        cache = (torch.randn(most * len(priors) + 1, 2, K, P, d, device="cuda") * 0.5).to(torch.bfloat16)
        table = torch.arange(most * len(priors), dtype=torch.int32, device="cuda").view(len(priors), most).contiguous()
        q = (torch.randn(sum(portions), H, d, device="cuda") * 0.5).to(torch.bfloat16)
        tiles, streams, row = [], [], 0
        for slot, (a, n) in enumerate(zip(priors, portions)):
            tiles += [[slot, row + i, a + i, min(16, n - i)] for i in range(0, n, 16)]
            tiles += [[slot, 0, 0, 0]] * (-len(tiles) % 16)
            streams += [(a + min(n, g + 256) - 1) // 64 + 1 for g in range(0, n, 256)]
            row += n
        return q, cache, table, torch.tensor(tiles, dtype=torch.int32, device="cuda"), streams

    def timed(q, cache, table, tiles, cut=None):
        out = torch.empty_like(q)
        more = {}
        if cut is not None:
            more = dict(segments=torch.from_numpy(cut[0]).cuda(), items=torch.from_numpy(cut[1]).cuda(), slots=cut[2])
        call = lambda: ops.prefill_attention_tc(q, cache, table, tiles, out, 0, 1 / math.sqrt(d), **more)
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(10):
                call()
        graph.replay()
        torch.cuda.synchronize()
        us = []
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            us.append(a.elapsed_time(b) * 100.0)
        return statistics.median(us)

    print(f"prefill_attention_tc_kernel<{d}>: one block per SM (148 heads, 256 query rows), us per launch")
    for prior in (0, 256, 768, 1792, 3840, 7936):
        q, cache, table, tiles, streams = case(148, 4, prior, 256)
        print(f"  stream of {streams[0]:4d} key tiles: {timed(q, cache, table, tiles):7.1f}")
    print(f"{heads} query heads, {kv_heads} kv heads: whole streams per block | the planner's cut")
    for prior, portion in ((0, 1024), (0, 2048), (0, 8192), (2048, 2048), (3840, 512), (32768, 128), (32768, 512),
                           ([0, 0, 0, 0], [512, 2048, 256, 1024]), ([0, 1024, 8192, 0], [1024, 512, 128, 512])):
        q, cache, table, tiles, streams = case(heads, kv_heads, prior, portion)
        several = isinstance(prior, list)
        flops = sum(4.0 * d * heads * sum(a + i + 1 for i in range(n))
                    for a, n in (zip(prior, portion) if several else [(prior, portion)]))
        whole = timed(q, cache, table, tiles)
        cut = plan_segments(streams, heads)
        name = f"{portion} behind {prior}" if several else f"{portion:5d} tokens behind {prior:5d}"
        line = f"  {name}: {whole:8.1f} us ({flops / whole / 1e6:6.0f} TFLOP/s)"
        if cut is not None:
            t = timed(q, cache, table, tiles, cut)
            line += f" | {t:8.1f} us ({flops / t / 1e6:6.0f} TFLOP/s; {len(cut[0])} blocks, {cut[2]} partial results merged)"
        else:
            line += " | as it is"
        print(line)
    return 0


def kernel_prompt_elementwise(cfg, rows):
    """The memory-bound kernels of a prompt step alone at the shape's widths, each beside a plain copy of the same
    bytes: ten launches replayed as a CUDA graph (data in L2), and the same with a 512 MB buffer written before
    each launch (data from memory; the time of the writes alone is subtracted)."""
    import statistics
    import torch
    from air_b200.csrc import ops
    E, H, K = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d, I, P, T = cfg.get("head_dim", E // H), cfg["intermediate_size"], 64, rows
    big = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")

    def graph_time(calls, reps=10):
        for c in calls:
            c()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(reps):
                for c in calls:
                    c()
        graph.replay()
        torch.cuda.synchronize()
        us = []
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            us.append(a.elapsed_time(b) * 1e3 / reps)
        return statistics.median(us)

    flush = lambda: big.zero_()
    t_flush = graph_time([flush])

    def report(name, f, nbytes):
        warm, cold = graph_time([f]), graph_time([flush, f]) - t_flush
        print(f"  {name:44s} {nbytes / 1e6:7.1f} MB  in L2 {warm:6.1f} us ({nbytes / warm / 1e6:5.2f} TB/s)  "
              f"from memory {cold:6.1f} us ({nbytes / cold / 1e6:5.2f} TB/s)", flush=True)
    print(f"{T} rows: hidden {E}, {H}/{K} heads of {d}, intermediate {I}")
    h = torch.randn(T, E, device="cuda")
    w = torch.ones(E, dtype=torch.bfloat16, device="cuda")
    x = torch.empty(T, E, dtype=torch.bfloat16, device="cuda")
    report("copy float32 -> bfloat16 [rows, hidden]", lambda: x.copy_(h), T * E * 6)
    report("add_rmsnorm, nothing to add", lambda: ops.add_rmsnorm(h, None, w, 1e-6, x), T * E * 6)
    delta = torch.randn(T, E, device="cuda")
    report("add_rmsnorm, a float32 delta", lambda: ops.add_rmsnorm(h, delta, w, 1e-6, x), T * E * 14)
    W = (H + 2 * K) * d
    qkv, bias = torch.randn(T, W, device="cuda"), torch.randn(W, device="cuda")
    table = torch.randn(T + 8, d, device="cuda")
    positions = torch.arange(T, dtype=torch.int32, device="cuda")
    seq = torch.zeros(T, dtype=torch.int32, device="cuda")
    pages = -(-T // P)
    bt = torch.arange(pages, dtype=torch.int32, device="cuda")[None, :].contiguous()
    q = torch.empty(T, H, d, dtype=torch.bfloat16, device="cuda")
    cache = torch.zeros(pages, 2, K, P, d, dtype=torch.bfloat16, device="cuda")
    report("bias + rotation + cache write", lambda: ops.qkv_rope_store(qkv, bias, table, positions, seq, bt, q, cache, H, K, d),
           T * W * 6)
    y = torch.empty(T, W, dtype=torch.bfloat16, device="cuda")
    report("copy float32 -> bfloat16 [rows, (H + 2K) d]", lambda: y.copy_(qkv), T * W * 6)
    gu = torch.randn(T, 2 * I, device="cuda").to(torch.bfloat16)
    act = torch.empty(T, I, dtype=torch.bfloat16, device="cuda")
    report("silu(gate) * up, blocks of 128", lambda: ops.silu_mul(gu, act, block=128), T * I * 6)
    z = torch.empty(T, 2 * I, dtype=torch.bfloat16, device="cuda")
    report("copy bfloat16 [rows, 2 x intermediate]", lambda: z.copy_(gu), T * I * 8)
    return 0


# ---------------------------------------------------------------------------------------------- a second design
# Bivizen beside the Qwen2 decoder at equal sizes (`--design bivizen`): layers that resemble a real model's, random
# weights.  A Bivizen model here alternates its three mixers: attention, delta, attention, gla.
def _bivizen(width, layers, heads, kv_heads, ff, vocab=32000):
    att = {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128,
                                          "rot": {"dims": 64, "base": 1e6}, "scale": 128 ** -0.5, "softcap": 30.0,
                                          "v_mix": True}}
    delta = {"type": "delta", "mixer": {"heads": heads, "kv_heads": heads // 2, "dim": 128, "vdim": 128, "conv": 4}}
    gla = {"type": "gla", "mixer": {"heads": heads // 2, "dim": 128, "vdim": 256, "tau": 16.0, "rank": 16}}
    mlp = {"kind": "dense", "ff": ff, "limit": 7.0}
    order = [att, delta, att, gla]
    return {"architecture": "Bivizen", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "layers": [dict(order[i % 4], mlp=mlp) for i in range(layers)]}


# Tomodra beside the Qwen2 decoder (`--design tomodra`): a latent-attention layer, one that reads its latent, and a
# layer of chunked attention with a sink, in turn; a latent of 512 + 64 per token, heads of 128 + 64 (values 128); 16
# experts of ff / 4 of which a token takes 2, and a shared expert of ff / 2, so that a token's feed-forward is as wide
# as the dense one beside it.
def _tomodra(width, layers, heads, kv_heads, ff, vocab=32000):
    def latent(i):
        m = {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "scale": 192 ** -0.5,
             "mask": {"size": 1024}, "rot": {"dims": 64, "base": 5e5}}
        if i % 3 == 1:
            m["kv_from"] = i - 1
        return {"type": "latent_attention", "mixer": m}
    att = {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128,
                                          "scale": 128 ** -0.5, "mask": {"size": 1024},
                                          "rot": {"dims": 64, "base": 1e4, "scaling": {"factor": 8.0, "original": 4096,
                                                                                      "fast": 32.0, "slow": 1.0}}}}
    mlp = {"kind": "moe", "expert": {"ff": ff // 4}, "router": {"experts": 16, "top": 2}, "shared": {"ff": ff // 2}}
    return {"architecture": "Tomodra", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "postln_alpha": 3.0,
            "layers": [dict(att if i % 3 == 2 else latent(i), mlp=mlp) for i in range(layers)]}


# Pefivik beside Tomodra, the closest of the other designs (attention over a latent, a mixture of experts), at equal
# width, heads, feed-forward and number of runs (`--design pefivik`): latent attention without positions over a latent
# of 512 with a sink and gates, an HGRN2 layer in every fourth place, dense PolyNorm feed-forwards and mixtures of 16
# experts of ff / 4 in 4 groups (2 take part, a token takes 2) with a shared expert of ff / 2 in turn; two of its layers
# run twice, so `layers` runs are layers - 2 layers' weights.
def _pefivik(width, layers, heads, kv_heads, ff, vocab=32000):
    latent = {"type": "latent_attention", "mixer": {"heads": heads, "dim": 128, "vdim": 128, "kv_rank": 512,
                                                    "scale": 128 ** -0.5}}
    hgrn = {"type": "hgrn2", "mixer": {"heads": heads, "dim": 128, "vdim": 128}}
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "expert": {"ff": ff // 4}, "router": {"experts": 16, "top": 2, "scale": 2.0,
                                                                "groups": {"count": 4, "keep": 2}},
           "shared": {"ff": ff // 2}}
    n = max(2, layers - 2)
    start = min(1, n - 2)
    return {"architecture": "Pefivik", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
            "logit_softcap": 50.0, "embedding": {"bigram": {"buckets": 65521, "mul_prev": 131, "mul_cur": 11}},
            "loop": {"start": start, "stop": start + 2, "times": 2},
            "layers": [dict(hgrn if i % 4 == 2 else latent, mlp=moe if i % 2 else dense) for i in range(n)]}


# Tabopel beside Tomodra, the closest of the other designs (grouped-query attention with a sink through the same mixer
# class, a mixture of experts), at equal width, heads and number of runs (`--design tabopel`): attention behind
# convolutions of four taps, attention with whole-vector norms and a soft cap, retention, attention, in turn, heads of
# 128; dense feed-forwards of 3 ff / 2 (as many weights as a gated one of ff) and mixtures of 16 experts of 3 ff / 8
# beside 2 identity experts, of which a token takes 4, in turn; two of its layers run twice, so `layers` runs are
# layers - 2 layers' weights.
def _tabopel(width, layers, heads, kv_heads, ff, vocab=32000):
    scaling = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}
    first = {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128, "conv": 4,
                                            "scale": 128 ** -0.5, "rot": {"dims": 128, "base": 5e5, "scaling": scaling}}}
    second = {"type": "attention_2", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128,
                                               "scale": 128 ** -0.5, "softcap": 50.0, "rot": {"dims": 64, "base": 5e5}}}
    ret = {"type": "retention", "mixer": {"heads": heads, "dim": 128, "vdim": 128, "rot": {"dims": 128, "base": 1e6},
                                          "decay": [1.0 - 2.0 ** (-5 - 5 * h / max(1, heads - 1)) for h in range(heads)]}}
    dense = {"kind": "dense", "ff": 3 * ff // 2}
    moe = {"kind": "moe", "expert": {"ff": 3 * ff // 8}, "router": {"experts": 16, "identity": 2, "top": 4}}
    n = max(2, layers - 2)
    start = min(1, n - 2)
    order = [first, second, ret, first]
    return {"architecture": "Tabopel", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": 8.0},
            "loop": {"start": start, "stop": start + 2, "times": 2},
            "layers": [dict(order[i % 4], mlp=moe if i % 2 else dense) for i in range(n)]}


def _qwen(width, layers, heads, kv_heads, ff, vocab=32000):
    return dict(_QWEN, num_hidden_layers=layers, hidden_size=width, num_attention_heads=heads,
                num_key_value_heads=kv_heads, intermediate_size=ff, rms_norm_eps=1e-5, max_window_layers=layers,
                vocab_size=vocab)


DESIGN_SIZES = {"2048": (2048, 8, 16, 4, 8192), "4096": (4096, 4, 32, 8, 14336)}


def design_model(cfg, args, torch, Entry, LAST):
    """Prefill of --prefill-tokens and decoding at --batch x --context for one configuration; the kernels' spans."""
    from air_b200.engine.engine import Engine, EngineConfig
    context, T, page = args.context or 2048, args.prefill_tokens, 64
    engine = Engine.from_random(cfg, seed=0, config=EngineConfig(
        dtype=torch.bfloat16, page_tokens=page, max_tokens=(args.batch + 1) * (context + 2 * page) + T + page,
        max_requests=args.batch + 1))
    randomize_cache(engine, torch)
    vocab = engine.model.spec.vocab_size
    prompt = torch.randint(0, vocab, (T,), generator=torch.Generator().manual_seed(7)).tolist()
    times = []
    for _ in range(2 + max(1, args.repeats)):
        torch.cuda.synchronize()
        time.sleep(args.prefill_pause_ms / 1e3)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        engine.step([Entry("p", prompt, [T - 1])])
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
        engine.finish("p")
    pre_ms = statistics.median(times[2:])
    requests = [f"r{i}" for i in range(args.batch)]
    dec, clocks, launches = decode_device(engine, requests, context, args.steps, args.warmup, max(1, min(3, args.repeats)),
                                          torch, Entry, LAST)
    dec_ms = statistics.median(dec)
    if args.timeline:
        prefill_timeline(engine, prompt, torch, Entry)
        decode_timeline(engine, requests, context, torch, Entry, LAST)
    engine.check_status()
    out = {"prefill_tokens": T, "prefill_ms": pre_ms, "prefill_tokens_per_s": T / (pre_ms / 1e3), "decode_batch": args.batch,
           "context": context, "decode_ms_per_step": dec_ms, "decode_tokens_per_s": args.batch / (dec_ms / 1e3),
           "weight_bytes": engine.model.weight_bytes(), "decode_launches": launches, "clocks": clocks}
    del engine
    torch.cuda.empty_cache()
    return out


def design_kernels(width, heads, kv_heads, ff, T, batch, context):
    """The new design's kernels alone at the layer's shapes beside the like kernel of the Qwen2 decoder, from memory
    (512 MB written before each launch, the writes' own time subtracted): microseconds, and the share of the measured
    copy rate (or, for the attention kernels, of the measured bf16 rate) that the algorithm's bytes (flops) make."""
    import torch
    from air_b200.csrc import ops
    from air_b200.parts.attention import TiledAttention
    from air_b200.parts.base import HostBatch
    pk = peaks()
    big = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")

    def graph_time(calls, reps=5):
        for c in calls:
            c()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(reps):
                for c in calls:
                    c()
        graph.replay()
        torch.cuda.synchronize()
        us = []
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            us.append(a.elapsed_time(b) * 1e3 / reps)
        return statistics.median(us)

    flush = lambda: big.zero_()
    t_flush = graph_time([flush])
    rows = []

    def report(name, f, nbytes=0, flops=0):
        us = graph_time([flush, f]) - t_flush
        frac = (nbytes / us / 1e3 / pk["hbm_gbs"]) if nbytes else (flops / us / 1e6 / pk["bf16_tflops"])
        rows.append({"kernel": name, "us": round(us, 1), "of": "copy rate" if nbytes else "bf16 rate", "frac": round(frac, 3)})
        print(f"  {name:58s} {us:8.1f} us  {frac:5.2f} of the measured {'copy' if nbytes else 'bf16'} rate", flush=True)

    E, H, G, d, I, P = width, heads, kv_heads, 128, ff, 64
    dev, f32, bf = "cuda", torch.float32, torch.bfloat16
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    for label, n_rows, entries, prior in (("prompt", T, [(0, T)], 0), ("decode", batch, [(context, 1)] * batch, context)):
        print(f"{label}: {n_rows} rows, width {E}, {H}/{G} heads of {d}, feed-forward {I}")
        S = len(entries)
        starts = [0]
        for _, n in entries:
            starts.append(starts[-1] + n)
        q_start = i32(starts)
        slots = i32(list(range(S)))
        positions = torch.cat([torch.arange(p, p + n, dtype=torch.int32) for p, n in entries]).to(dev)
        seq = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, (_, n) in enumerate(entries)]).to(dev)
        blocks = -(-(prior + T) // P)
        bt = torch.arange(S * blocks, dtype=torch.int32, device=dev).view(S, blocks).contiguous()
        cache = torch.randn(S * blocks, 2, G, P, d, device=dev).to(bf)
        R = n_rows
        # the norm with the two scaled outputs of the layer before it | add + norm
        h, a, b = (torch.randn(R, E, device=dev) for _ in range(3))
        sa, sb, w = torch.randn(E, device=dev), torch.randn(E, device=dev), torch.ones(E, dtype=bf, device=dev)
        x = torch.empty(R, E, dtype=bf, device=dev)
        report("scaled_norm (stream + 2 scaled terms, norm)", lambda: ops.scaled_norm(h, [(a, sa), (b, sb)], w, 1e-5, x), R * E * 18)
        report("  Qwen2: add_rmsnorm (stream + 1 term, norm)", lambda: ops.add_rmsnorm(h, a, w, 1e-5, x), R * E * 14)
        # bias, rotation, value mixing, gate, cache write | bias, rotation, cache write
        W = (H + 2 * G) * d + H
        proj, bias = torch.randn(R, W, device=dev), torch.randn(W, device=dev)
        freq = torch.rand(32, device=dev)
        qo, go = torch.empty(R, H, d, dtype=bf, device=dev), torch.empty(R, H, device=dev)
        vf, lam = torch.randn(R, G * d, device=dev), torch.tensor([0.4], device=dev)
        flat = cache.view(cache.shape[0], -1)
        report("qkv_prepare (bias, rotation, value mix, gates, cache write)",
               lambda: ops.qkv_prepare(proj, bias, freq, positions, seq, bt, qo, flat, G, d, P, gate_out=go, v_first=vf,
                                       v_mode=2, v_lambda=lam), R * (W * 4 + (H + 2 * G) * d * 2 + G * d * 4))
        qkv, table = proj[:, :W - H].contiguous(), torch.randn(prior + T + 8, d, device=dev)
        report("  Qwen2: qkv_rope_store", lambda: ops.qkv_rope_store(qkv, bias[:W - H].contiguous(), table, positions, seq,
                                                                      bt, qo, cache, H, G, d), R * (W - H) * 6)
        # attention
        out = torch.empty_like(qo)
        if label == "prompt":
            planner = type("P", (TiledAttention,), {"heads": H, "window": None})()
            plan = planner.plan(HostBatch(counts=[T], lengths=[0], slots=[0], q_start=[0, T]))
            tiles = i32(plan.arrays["tiles"].tolist())
            fl = 4 * H * d * (T * (T + 1) // 2)
            report("prefill_attention_tc with a soft cap", lambda: ops.prefill_attention_tc(qo, cache, bt, tiles, out, None, d ** -0.5, softcap=30.0), flops=fl)
            report("  Qwen2: prefill_attention_tc", lambda: ops.prefill_attention_tc(qo, cache, bt, tiles, out, None, d ** -0.5), flops=fl)
        else:
            nb = batch * context * 2 * G * d * 2
            report("decode_attention with a soft cap", lambda: ops.decode_attention(qo, cache, bt, seq, positions, out, None, d ** -0.5, softcap=30.0), nb)
            report("  Qwen2: decode_attention", lambda: ops.decode_attention(qo, cache, bt, seq, positions, out, None, d ** -0.5), nb)
        report("head_gate", lambda: ops.head_gate(out, go, seq), R * H * d * 4)
        # the state mixers: convolution, scans, gated norm (no like kernel in the Qwen2 decoder)
        Gd, Hs = H // 2, H
        C = 2 * Gd * d + Hs * d
        xs, cw = torch.randn(R, C + 2 * Hs, device=dev), torch.randn(C, 4, device=dev)
        tail, y = torch.zeros(S, C, 3, device=dev), torch.empty(R, C, device=dev)
        longest = max(n for _, n in entries)
        report("short_conv_silu (4 taps)", lambda: ops.short_conv_silu(xs[:, :C], cw, tail, y, q_start, slots, longest),
               R * C * 8 + (S * C * 24 if label == "decode" else 0))
        state, o = torch.zeros(S, Hs, d, d, device=dev), torch.empty(R, Hs, d, device=dev)
        al, dtb = torch.zeros(Hs, device=dev), torch.zeros(Hs, device=dev)
        scan_bytes = R * (C + Hs * d) * 4 + S * Hs * d * d * 8
        report("linear_scan, delta rule", lambda: ops.linear_scan(
            ops.SCAN_DELTA, y[:, :Gd * d], y[:, Gd * d:2 * Gd * d], y[:, 2 * Gd * d:], xs[:, C:C + Hs], state, o, q_start,
            slots, seq, q_scale=d ** -0.5, beta=xs[:, C + Hs:], a_log=al, dt_bias=dtb, unit=True), scan_bytes)
        Hg, dvg = H // 2, 256
        qg, vg, zg = torch.randn(R, 2 * Hg * d, device=dev), torch.randn(R, Hg * dvg, device=dev), torch.randn(R, Hg * d, device=dev)
        sg, og = torch.zeros(S, Hg, d, dvg, device=dev), torch.empty(R, Hg, dvg, device=dev)
        report("linear_scan, gated linear attention", lambda: ops.linear_scan(
            ops.SCAN_GLA, qg[:, :Hg * d], qg[:, Hg * d:], vg, zg, sg, og, q_start, slots, seq, q_scale=d ** -0.5, tau=16.0),
            R * (3 * Hg * d + 2 * Hg * dvg) * 4 + S * Hg * d * dvg * 8)
        gate, nw = torch.randn(R, Hs * d, device=dev), torch.ones(d, device=dev)
        yo = torch.empty(R, Hs * d, dtype=bf, device=dev)
        report("gated_rmsnorm", lambda: ops.gated_rmsnorm(o, gate, nw, 1e-5, yo, seq), R * Hs * d * 10)
        # the feed-forward's activation
        gu32, act = torch.randn(R, 2 * I, device=dev), torch.empty(R, I, dtype=bf, device=dev)
        report("glu with limits (float32 product in)", lambda: ops.glu(gu32, act, block=128, alpha=1.702, limit=7.0, shift=1.0), R * I * 10)
        gu16 = gu32.to(bf)
        report("  Qwen2: silu_mul (bfloat16 product in)", lambda: ops.silu_mul(gu16, act, block=128), R * I * 6)
        del cache
    return rows


def tomodra_kernels(width, heads, kv_heads, ff, T, batch, context):
    """Tomodra's kernels alone at the layer's shapes beside the like kernel of the Qwen2 decoder, from memory (512 MB
    written before each launch, the writes' own time subtracted): microseconds, and the share of the measured copy
    rate (bytes) or of the measured bf16 rate (flops) that the algorithm's bytes or flops make."""
    import torch
    from types import SimpleNamespace
    from air_b200.csrc import ops
    from air_b200.parts.base import HostBatch, Runtime
    from air_b200.parts.gathered_attention import PortionAttention
    from air_b200.parts.rope import bent_frequencies
    pk = peaks()
    big = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")

    def graph_time(calls, reps=5):
        for c in calls:
            c()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(reps):
                for c in calls:
                    c()
        graph.replay()
        torch.cuda.synchronize()
        us = []
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            us.append(a.elapsed_time(b) * 1e3 / reps)
        return statistics.median(us)

    flush = lambda: big.zero_()
    t_flush = graph_time([flush])
    rows = []

    def report(name, f, nbytes=0, flops=0):
        us = graph_time([flush, f]) - t_flush
        frac = (nbytes / us / 1e3 / pk["hbm_gbs"]) if nbytes else (flops / us / 1e6 / pk["bf16_tflops"])
        rows.append({"kernel": name, "us": round(us, 1), "of": "copy rate" if nbytes else "bf16 rate", "frac": round(frac, 3)})
        print(f"  {name:64s} {us:8.1f} us  {frac:5.2f} of the measured {'copy' if nbytes else 'bf16'} rate", flush=True)

    E, H, G, d, P = width, heads, kv_heads, 128, 64
    R, rot, window = 512, 64, 1024
    n_exp, top, F = 16, 2, ff // 4
    dev, f32, bf = "cuda", torch.float32, torch.bfloat16
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    freq = bent_frequencies(rot, 5e5, None)[0].to(dev)
    for label, n_rows, entries in (("prompt", T, [(0, T)]), ("decode", batch, [(context, 1)] * batch)):
        print(f"{label}: {n_rows} rows, width {E}, {H} heads, latent {R} + {rot}, window {window}, {n_exp} experts of {F}, top {top}")
        S = len(entries)
        positions = torch.cat([torch.arange(p, p + n, dtype=torch.int32) for p, n in entries]).to(dev)
        seq = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, (_, n) in enumerate(entries)]).to(dev)
        per_request = -(-(max(p + n for p, n in entries)) // P)
        bt = torch.arange(S * per_request, dtype=torch.int32, device=dev).view(S, per_request).contiguous()
        N = n_rows
        # ---- the norm behind the sum, beside the norm before the sub-layer
        h, delta = torch.randn(N, E, device=dev), torch.randn(N, E, device=dev)
        w, x16 = torch.ones(E, device=dev, dtype=bf), torch.empty(N, E, device=dev, dtype=bf)
        report("post_norm (stream, a float32 sum in; stream and rows out)", lambda: ops.post_norm(h, 3.0, delta, None, None, w, 1e-5, x16), N * E * 14)
        report("  Qwen2: add_rmsnorm", lambda: ops.add_rmsnorm(h, delta, w, 1e-5, x16), N * E * 14)
        # ---- from the first projection to queries and the latent's pages
        proj = torch.randn(N, H * (d + rot) + R + rot, device=dev)
        cw = torch.ones(R, device=dev)
        rows_ = torch.zeros(S * per_request, P, R + rot, device=dev, dtype=bf).normal_(0, 0.5)
        q_plain, q_full = torch.empty(N, H, d, device=dev, dtype=bf), torch.empty(N, H, R + rot, device=dev)
        report("latent_prepare (norm of the latent, rotation, page write)", lambda: ops.latent_prepare(proj, cw, 1e-5, freq, positions, seq, bt, q_plain, q_full, rows_, True),
               N * (proj.shape[1] * 4 + H * d * 2 + H * rot * 4 + (R + rot) * 2))
        Wq = (H + 2 * G) * d
        qkv = torch.randn(N, Wq, device=dev)
        qn, q16 = torch.ones(d, device=dev), torch.empty(N, H, d, device=dev, dtype=bf)
        kvc = torch.zeros(S * per_request, 2 * G * P * d, device=dev, dtype=bf).normal_(0, 0.5)
        f2 = bent_frequencies(64, 1e4, {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0})[0].to(dev)
        report("qk_normed_prepare (norm per head, rotation, page write)", lambda: ops.qk_normed_prepare(qkv, qn, qn, 1e-5, f2, "neighbours", 1.2, positions, seq, bt, q16, kvc, G, d, P),
               N * Wq * 6)
        table = torch.randn(context + T + 8, d, device=dev)
        kv5 = kvc.view(-1, 2, G, P, d)
        report("  Qwen2: qkv_rope_store", lambda: ops.qkv_rope_store(qkv, None, table, positions, seq, bt, q16, kv5, H, G, d), N * Wq * 6)
        # ---- the products per head around latent attention
        uk_t = torch.randn(H, R, d, device=dev, dtype=bf)
        report("grouped product: queries through the key expansion", lambda: ops.grouped_gemm(q_plain, uk_t, q_full, R, d, lda=H * d, ldo=H * (R + rot), groups=H, a_group_stride=d, o_group_stride=R + rot, a_local=True, o_local=True, rows_per_group=N),
               flops=2 * N * H * d * R)
        # ---- attention
        summed = torch.empty(N, H, R, device=dev, dtype=bf)
        out16 = torch.empty(N, H, d, device=dev, dtype=bf)
        if label == "decode":
            keys = min(window, context + 1)
            report("grouped_attention, latent rows (all heads read a row once)", lambda: ops.grouped_attention(q_full, rows_, bt, seq, positions, summed, window, 0.07, latent=True),
                   batch * keys * (R + rot) * 2)
            sink = torch.zeros(H, device=dev)
            report("grouped_attention, keys and values per head, chunk, sink", lambda: ops.grouped_attention(q16, kvc, bt, seq, positions, out16, None, 0.09, kv_heads=G, page_tokens=P, chunk=window, sink=sink),
                   batch * (context % window + 1) * 2 * G * d * 2)
            report("  Qwen2: decode_attention (all keys)", lambda: ops.decode_attention(q16, kv5, bt, seq, positions, out16, None, 0.09),
                   batch * (context + 1) * 2 * G * d * 2)
        else:
            class Road(PortionAttention):
                rt = Runtime(device=torch.device(dev), dtype=bf, page_tokens=P)
                chunk, sinks = None, None
            road = Road()
            road.heads, road.window, road.scale = H, window, 0.07
            plan = road.plan(HostBatch(counts=[T], lengths=[0], slots=[0], q_start=[0, T]))
            ctx = SimpleNamespace(plans={road.plan_key(): SimpleNamespace(small_seq=i32(plan.arrays["small_seq"]), **plan.values)},
                                  token_seq=seq, positions=positions)
            pairs_seen = sum(min(window, t + 1) for t in range(T))
            t0 = time.time()
            us = []
            for _ in range(5):
                flush()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                road.attend(q_full, rows_, bt, ctx, summed, latent=True)
                b.record()
                torch.cuda.synchronize()
                us.append(a.elapsed_time(b) * 1e3)
            us = statistics.median(us[1:])
            fl = 2 * pairs_seen * H * (2 * R + rot)
            rows.append({"kernel": "portion attention over latent rows (gather, product, softmax, product)", "us": round(us, 1), "of": "bf16 rate", "frac": round(fl / us / 1e6 / pk["bf16_tflops"], 3)})
            print(f"  {'portion attention over latent rows (gather, 2 products, softmax), launched from the host':64s} {us:8.1f} us  {fl / us / 1e6 / pk['bf16_tflops']:5.2f} of the measured bf16 rate (the flops of the keys that are seen)")
            tiles = i32([[0, 16 * i, 16 * i, 16] for i in range(T // 16)])
            report("  Qwen2: prefill_attention_tc (all keys, heads of 128)", lambda: ops.prefill_attention_tc(q16, kv5, bt, tiles, out16, None, 0.09),
                   flops=2 * (T * (T + 1) // 2) * H * 2 * d)
        # ---- the experts
        x = torch.randn(N, E, device=dev, dtype=bf)
        z = torch.randn(N, 24, device=dev)
        expert = torch.empty(N, top, dtype=torch.int32, device=dev)
        weight, gate = torch.empty(N, top, device=dev), torch.empty(N, device=dev)
        pairs = N * top
        start, slots_ = torch.empty(n_exp + 1, dtype=torch.int32, device=dev), torch.empty(pairs, dtype=torch.int32, device=dev)
        tiles_, count = torch.empty(pairs // 64 + n_exp, 2, dtype=torch.int32, device=dev), torch.empty(1, dtype=torch.int32, device=dev)
        report("moe_route + moe_sort", lambda: (ops.moe_route(z, n_exp, top, expert, weight, gate, has_gate=True), ops.moe_sort(expert, n_exp, start, slots_, tiles_, count)), N * 24 * 4 + pairs * 16)
        gate_up, down = torch.randn(n_exp, 2 * F, E, device=dev, dtype=bf) * 0.02, torch.randn(n_exp, E, F, device=dev, dtype=bf) * 0.02
        act, y = torch.empty(pairs, F, device=dev, dtype=bf), torch.empty(top, N, E, device=dev)
        if label == "decode":
            used = len(set(expert.flatten().tolist()))
            report(f"grouped product: gate, up and activation of {used} experts", lambda: ops.grouped_gemm(x, gate_up, act, F, E, lda=E, ldo=F, groups=n_exp, a_index=slots_, a_div=top, a_scale=weight.view(-1), start=start, tiles=tiles_, num_tiles=count, silu_mul=True, gate_block=128),
                   used * 2 * F * E * 2)
            report(f"grouped product: down of {used} experts", lambda: ops.grouped_gemm(act, down, y, E, F, lda=F, ldo=E, groups=n_exp, o_index=slots_, o_div=top, o_part_stride=N * E, start=start, tiles=tiles_, num_tiles=count),
                   used * F * E * 2)
            dense = torch.randn(2 * ff, E, device=dev, dtype=bf) * 0.02
            dact = torch.empty(N, ff, device=dev, dtype=bf)
            report("  Qwen2: gate, up and activation (gemm_tc, dense, as wide as 4 experts)", lambda: ops.gemm_tc(x, dense, dact, 256, ops.EPI_SILU), 2 * ff * E * 2)
        else:
            xs = torch.empty(pairs, E, device=dev, dtype=bf)
            ends = start[1:].clone()
            report("experts: rows in order, library grouped product, activation", lambda: (ops.rows_by_index(x, slots_, top, weight.view(-1), xs), ops.silu_mul(torch._grouped_mm(xs, gate_up.transpose(1, 2), offs=ends), act, block=128)),
                   flops=2 * pairs * 2 * F * E)
            report("experts: library grouped product for down, rows back to planes", lambda: ops.planes_by_index(torch._grouped_mm(act, down.transpose(1, 2), offs=ends), slots_, top, y),
                   flops=2 * pairs * F * E)
            dense = torch.randn(2 * ff, E, device=dev, dtype=bf) * 0.02
            dact = torch.empty(N, ff, device=dev, dtype=bf)
            report("  Qwen2: gate, up and activation (gemm_tc, dense, the same flops)", lambda: ops.gemm_tc(x, dense, dact, 256, ops.EPI_SILU), flops=2 * N * 2 * ff * E)
    return rows


def pefivik_kernels(width, heads, kv_heads, ff, T, batch, context):
    """Pefivik's kernels alone at the layer's shapes, each beside the like kernel of Tomodra, Bivizen or the Qwen2
    decoder, from memory (512 MB written before each launch, the writes' own time subtracted): microseconds, and the
    share of the measured copy rate (bytes) or of the measured bf16 rate (flops) that the algorithm's bytes or flops
    make."""
    import torch
    from air_b200.csrc import ops
    pk = peaks()
    big = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")

    def graph_time(calls, reps=5):
        for c in calls:
            c()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(reps):
                for c in calls:
                    c()
        graph.replay()
        torch.cuda.synchronize()
        us = []
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            us.append(a.elapsed_time(b) * 1e3 / reps)
        return statistics.median(us)

    flush = lambda: big.zero_()
    t_flush = graph_time([flush])
    rows = []

    def report(name, f, nbytes=0, flops=0):
        us = graph_time([flush, f]) - t_flush
        frac = (nbytes / us / 1e3 / pk["hbm_gbs"]) if nbytes else (flops / us / 1e6 / pk["bf16_tflops"])
        rows.append({"kernel": name, "us": round(us, 1), "of": "copy rate" if nbytes else "bf16 rate", "frac": round(frac, 3)})
        print(f"  {name:66s} {us:8.1f} us  {frac:5.2f} of the measured {'copy' if nbytes else 'bf16'} rate", flush=True)

    E, H, d, P, R = width, heads, 128, 64, 512
    n_exp, top, F = 16, 2, ff // 4
    dev, bf = "cuda", torch.bfloat16
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    for label, N, entries in (("prompt", T, [(0, T)]), ("decode", batch, [(context, 1)] * batch)):
        print(f"{label}: {N} rows, width {E}, {H} heads of {d}, latent {R}, {n_exp} experts of {F} in 4 groups, top {top}")
        S = len(entries)
        starts = [0]
        for _, n in entries:
            starts.append(starts[-1] + n)
        q_start, slots = i32(starts), i32(list(range(S)))
        positions = torch.cat([torch.arange(p, p + n, dtype=torch.int32) for p, n in entries]).to(dev)
        seq = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, (_, n) in enumerate(entries)]).to(dev)
        per_request = -(-(max(p + n for p, n in entries)) // P)
        bt = torch.arange(S * per_request, dtype=torch.int32, device=dev).view(S, per_request).contiguous()
        # ---- the embedding with its table of pairs, beside the plain one
        V, buckets = 32000, 65521
        table, pairs = torch.randn(V, E, device=dev, dtype=bf), torch.randn(buckets + 1, E, device=dev, dtype=bf)
        ids = torch.randint(0, V, (N,), dtype=torch.int32, device=dev)
        previous, resolved = torch.zeros(S, 1, dtype=torch.int32, device=dev), torch.empty(N, dtype=torch.int32, device=dev)
        h, h2 = torch.empty(N, E, device=dev), torch.empty(N, E, device=dev)
        report("bigram_embedding (two rows in, the stream and a copy out) + remember_tokens",
               lambda: (ops.bigram_embedding(table, pairs, ids, positions, seq, previous, h, h2, resolved, buckets, 131, 11),
                        ops.remember_tokens(resolved, q_start, slots, previous, S)), N * E * 12)
        report("  Qwen2: embedding", lambda: ops.embedding(table, ids, h), N * E * 6)
        # ---- what a pass adds, and the norm that completes the stream with scaled sums
        row, delta = torch.randn(E, device=dev), torch.randn(N, E, device=dev)
        report("stream_add (the embedding's output again and a row)", lambda: ops.stream_add(h, h2, row), N * E * 12)
        sc, w, x16 = torch.full((E,), 0.5, device=dev), torch.ones(E, device=dev, dtype=bf), torch.empty(N, E, device=dev, dtype=bf)
        planes = torch.randn(top, N, E, device=dev)
        report("scaled_norm (stream + m x one term, scalar norm)", lambda: ops.scaled_norm(h, [(delta, sc)], w, 1e-5, x16), N * E * 14)
        report("scaled_norm (stream + m x (experts' planes + shared expert))", lambda: ops.scaled_norm(h, [(planes, sc), (delta, sc)], w, 1e-5, x16), N * E * (14 + 4 * top))
        report("  Tomodra: post_norm (stream + planes + shared expert)", lambda: ops.post_norm(h, 3.0, planes, delta, None, w, 1e-5, x16), N * E * (14 + 4 * top))
        report("  Qwen2: add_rmsnorm", lambda: ops.add_rmsnorm(h, delta, w, 1e-5, x16), N * E * 14)
        # ---- from the first projection to queries, gates and the latent's pages
        cols = -(-(H * d + R + H) // 8) * 8
        proj, cw = torch.randn(N, cols, device=dev), torch.ones(R, device=dev)
        rows_ = torch.zeros(S * per_request, P, R, device=dev, dtype=bf).normal_(0, 0.5)
        q_plain, q_full = torch.empty(N, H, d, device=dev, dtype=bf), torch.empty(N, H, R, device=dev)
        gate = torch.empty(N, H, device=dev)
        report("latent_prepare (norm of the latent, gates, page write; no rotation)",
               lambda: ops.latent_prepare(proj, cw, 1e-5, None, positions, seq, bt, q_plain, q_full, rows_, True, gate_out=gate, gate_column=H * d + R),
               N * (cols * 4 + H * d * 2 + R * 2 + H * 4))
        freq = torch.rand(32, device=dev, dtype=torch.float64)
        proj_t = torch.randn(N, H * (d + 64) + R + 64, device=dev)
        rows_t = torch.zeros(S * per_request, P, R + 64, device=dev, dtype=bf).normal_(0, 0.5)
        q_full_t = torch.empty(N, H, R + 64, device=dev)
        report("  Tomodra: latent_prepare (norm, rotation of 64, page write)",
               lambda: ops.latent_prepare(proj_t, cw, 1e-5, freq, positions, seq, bt, q_plain, q_full_t, rows_t, True),
               N * (proj_t.shape[1] * 4 + H * d * 2 + H * 64 * 4 + (R + 64) * 2))
        out16 = torch.empty(N, H, d, device=dev, dtype=bf)
        sums16, uv = torch.randn(N, H, R, device=dev).to(bf), torch.randn(H, d, R, device=dev, dtype=bf) * 0.05
        report("grouped product: value expansion per head, the gate in its epilogue", lambda: ops.grouped_gemm(sums16, uv, out16, d, R, lda=H * R, ldo=H * d, groups=H, a_group_stride=R, o_group_stride=d, a_local=True, o_local=True, rows_per_group=N, o_scale=gate, o_scale_ld=H),
               flops=2 * N * H * d * R)
        report("  Tomodra: the same product without a gate", lambda: ops.grouped_gemm(sums16, uv, out16, d, R, lda=H * R, ldo=H * d, groups=H, a_group_stride=R, o_group_stride=d, a_local=True, o_local=True, rows_per_group=N),
               flops=2 * N * H * d * R)
        # ---- attention over the latent's rows
        summed = torch.empty(N, H, R, device=dev, dtype=bf)
        sink = torch.zeros(H, device=dev)
        if label == "decode":
            report("grouped_attention, latent rows of 512, all keys, sink", lambda: ops.grouped_attention(q_full, rows_, bt, seq, positions, summed, None, 0.09, latent=True, sink=sink),
                   batch * (context + 1) * R * 2)
            summed_t = torch.empty(N, H, R, device=dev, dtype=bf)
            report("  Tomodra: grouped_attention, latent rows of 576, window 1,024", lambda: ops.grouped_attention(q_full_t, rows_t, bt, seq, positions, summed_t, 1024, 0.07, latent=True),
                   batch * min(1024, context + 1) * (R + 64) * 2)
        # ---- the state mixer: what the scan reads, the scan, the norm per head
        Hs = H
        xs = torch.randn(N, 3 * Hs * d, device=dev)
        state, o = torch.zeros(S, Hs, d, d, device=dev), torch.empty(N, Hs, d, device=dev)
        low, fb = torch.rand(Hs * d, device=dev) * 0.9, torch.zeros(Hs * d, device=dev)
        scan_bytes = N * 4 * Hs * d * 4 + S * Hs * d * d * 8
        report("linear_scan, HGRN2 (gate, lower bound, silu in the preparation)", lambda: ops.linear_scan(
            ops.SCAN_HGRN, xs[:, :Hs * d], None, xs[:, 2 * Hs * d:], xs[:, Hs * d:2 * Hs * d], state, o, q_start, slots, seq,
            lower=low, gate_bias=fb), scan_bytes)
        xg = torch.randn(N, 4 * Hs * d, device=dev)
        report("  Bivizen: linear_scan, gated linear attention (same sizes)", lambda: ops.linear_scan(
            ops.SCAN_GLA, xg[:, :Hs * d], xg[:, Hs * d:2 * Hs * d], xg[:, 2 * Hs * d:3 * Hs * d], xg[:, 3 * Hs * d:], state, o,
            q_start, slots, seq, q_scale=d ** -0.5, tau=16.0), scan_bytes + N * Hs * d * 4)
        nw, yo = torch.ones(d, device=dev), torch.empty(N, Hs * d, dtype=bf, device=dev)
        report("gated_rmsnorm without a gate (norm per head)", lambda: ops.gated_rmsnorm(o, None, nw, 1e-5, yo, seq), N * Hs * d * 6)
        report("  Bivizen: gated_rmsnorm", lambda: ops.gated_rmsnorm(o, xg[:, :Hs * d], nw, 1e-5, yo, seq), N * Hs * d * 10)
        # ---- the dense feed-forward's activation
        z, ub = torch.randn(N, ff, device=dev), torch.randn(ff, device=dev)
        act = torch.empty(N, ff + 8, device=dev, dtype=bf)
        report("polynorm (float32 product and bias in, three norms)", lambda: ops.polynorm(z, ub, (1.0, 0.4, -0.1, 0.0), 1e-5, act, ff), N * ff * 6)
        gu16, act2 = torch.randn(N, 2 * ff, device=dev).to(bf), torch.empty(N, ff, device=dev, dtype=bf)
        report("  Qwen2: silu_mul (bfloat16 product in)", lambda: ops.silu_mul(gu16, act2, block=128), N * ff * 6)
        gu32 = torch.randn(N, 2 * ff, device=dev)
        report("  Bivizen: glu with limits (float32 product in)", lambda: ops.glu(gu32, act2, block=128, alpha=1.702, limit=7.0, shift=1.0), N * ff * 10)
        # ---- the experts
        x = torch.randn(N, E, device=dev, dtype=bf)
        zr = torch.randn(N, 16, device=dev)
        expert = torch.empty(N, top, dtype=torch.int32, device=dev)
        weight = torch.empty(N, top, device=dev)
        pairs_n = N * top
        start, slots_ = torch.empty(n_exp + 1, dtype=torch.int32, device=dev), torch.empty(pairs_n, dtype=torch.int32, device=dev)
        tiles_, count = torch.empty(pairs_n // 64 + n_exp, 2, dtype=torch.int32, device=dev), torch.empty(1, dtype=torch.int32, device=dev)
        report("moe_route among the best 2 of 4 groups", lambda: ops.moe_route(zr, n_exp, top, expert, weight, None, renormalize=True, groups=4, keep=2, route_scale=1.5, norm_eps=1e-20), N * 16 * 4 + pairs_n * 8)
        report("  Tomodra: moe_route", lambda: ops.moe_route(zr, n_exp, top, expert, weight, None), N * 16 * 4 + pairs_n * 8)
        ops.moe_route(zr, n_exp, top, expert, weight, None, renormalize=True, groups=4, keep=2, route_scale=1.5, norm_eps=1e-20)
        ops.moe_sort(expert, n_exp, start, slots_, tiles_, count)
        down = torch.randn(n_exp, E, F, device=dev, dtype=bf) * 0.02
        acts, y = torch.randn(pairs_n, F, device=dev, dtype=bf), torch.empty(top, N, E, device=dev)
        if label == "decode":
            used = len(set(expert.flatten().tolist()))
            report(f"grouped product: down of {used} experts, the weight on the output", lambda: ops.grouped_gemm(acts, down, y, E, F, lda=F, ldo=E, groups=n_exp, o_index=slots_, o_div=top, o_part_stride=N * E, start=start, tiles=tiles_, num_tiles=count, o_scale=weight.view(-1)),
                   used * F * E * 2)
            report(f"  Tomodra: grouped product: down of {used} experts", lambda: ops.grouped_gemm(acts, down, y, E, F, lda=F, ldo=E, groups=n_exp, o_index=slots_, o_div=top, o_part_stride=N * E, start=start, tiles=tiles_, num_tiles=count),
                   used * F * E * 2)
        else:
            ends = start[1:].clone()
            report("experts: library grouped product for down, weighted rows back to planes", lambda: ops.planes_by_index(torch._grouped_mm(acts, down.transpose(1, 2), offs=ends), slots_, top, y, scale=weight.view(-1)),
                   flops=2 * pairs_n * F * E)
            report("  Tomodra: the same without the weight", lambda: ops.planes_by_index(torch._grouped_mm(acts, down.transpose(1, 2), offs=ends), slots_, top, y),
                   flops=2 * pairs_n * F * E)
    return rows


def tabopel_kernels(width, heads, kv_heads, ff, T, batch, context):
    """Tabopel's kernels alone at the layer's shapes, each beside the like kernel of Tomodra, Pefivik, Bivizen or the
    Qwen2 decoder, from memory (512 MB written before each launch, the writes' own time subtracted): microseconds, and
    the share of the measured copy rate (bytes) or of the measured bf16 rate (flops) that the algorithm's bytes or
    flops make."""
    import torch
    from air_b200.csrc import ops
    pk = peaks()
    big = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")

    def graph_time(calls, reps=5):
        for c in calls:
            c()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(reps):
                for c in calls:
                    c()
        graph.replay()
        torch.cuda.synchronize()
        us = []
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            us.append(a.elapsed_time(b) * 1e3 / reps)
        return statistics.median(us)

    flush = lambda: big.zero_()
    t_flush = graph_time([flush])
    rows = []

    def report(name, f, nbytes=0, flops=0):
        us = graph_time([flush, f]) - t_flush
        frac = (nbytes / us / 1e3 / pk["hbm_gbs"]) if nbytes else (flops / us / 1e6 / pk["bf16_tflops"])
        rows.append({"kernel": name, "us": round(us, 1), "of": "copy rate" if nbytes else "bf16 rate", "frac": round(frac, 3)})
        print(f"  {name:70s} {us:8.1f} us  {frac:5.2f} of the measured {'copy' if nbytes else 'bf16'} rate", flush=True)

    E, H, G, d, P = width, heads, kv_heads, 128, 64
    n_exp, ident, top, F = 16, 2, 4, 3 * ff // 8
    dev, bf, f32 = "cuda", torch.bfloat16, torch.float32
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    for label, N, entries in (("prompt", T, [(0, T)]), ("decode", batch, [(context, 1)] * batch)):
        print(f"{label}: {N} rows, width {E}, {H}/{G} heads of {d}, {n_exp} + {ident} experts of {F}, top {top}")
        S = len(entries)
        starts = [0]
        for _, n in entries:
            starts.append(starts[-1] + n)
        q_start, slots = i32(starts), i32(list(range(S)))
        positions = torch.cat([torch.arange(p, p + n, dtype=torch.int32) for p, n in entries]).to(dev)
        seq = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, (_, n) in enumerate(entries)]).to(dev)
        per_request = -(-(max(p + n for p, n in entries)) // P)
        bt = torch.arange(S * per_request, dtype=torch.int32, device=dev).view(S, per_request).contiguous()
        longest = max(n for _, n in entries)
        # ---- the norm behind a sub-layer, the sum and the norm ahead of the next one, beside the sums with one norm
        h, a = torch.randn(N, E, device=dev), torch.randn(N, E, device=dev)
        parts4 = torch.randn(top, N, E, device=dev)
        wb, w = torch.rand(E, device=dev) + 0.5, torch.rand(E, device=dev) + 0.5
        wbf = w.to(bf)
        x = torch.empty(N, E, dtype=bf, device=dev)
        report("normed_add_norm (norm of the term, stream + term, norm)", lambda: ops.normed_add_norm(h, a, wb, 1e-6, w, 1e-6, x), N * E * 14)
        report("  Qwen2: add_rmsnorm (stream + term, norm)", lambda: ops.add_rmsnorm(h, a, wbf, 1e-6, x), N * E * 14)
        report("normed_add_norm with the experts' four planes", lambda: ops.normed_add_norm(h, parts4, wb, 1e-6, w, 1e-6, x), N * E * (10 + 4 * top))
        report("  Pefivik: scaled_norm with two planes and the shared expert",
               lambda: ops.scaled_norm(h, [(parts4[:2], wb), (a, wb)], wbf, 1e-6, x), N * E * (10 + 12))
        # ---- the convolutions behind the projections, beside the delta rule's (with SiLU)
        C = (H + G) * d + G * d
        proj = torch.randn(N, C + H * d, device=dev)
        cw, tail = torch.randn(C, 4, device=dev), torch.zeros(S, C, 3, device=dev)
        y = torch.empty(N, C, device=dev)
        report("short_conv, 4 taps, no activation (q, k, v)", lambda: ops.short_conv_silu(proj[:, :C], cw, tail, y, q_start, slots, longest, act=False), N * C * 8)
        report("  Bivizen: short_conv_silu", lambda: ops.short_conv_silu(proj[:, :C], cw, tail, y, q_start, slots, longest), N * C * 8)
        # ---- bias, whole-vector norm, rotation, page write, beside the norm per head
        pages = torch.zeros(S * per_request, G * P * 2 * d, dtype=bf, device=dev)
        qo = torch.empty(N, H, d, dtype=bf, device=dev)
        freq = torch.rand(d // 2, dtype=torch.float64, device=dev)
        bias = torch.randn(C, device=dev)
        qw, kw = torch.rand(H * d, device=dev), torch.rand(G * d, device=dev)
        nbytes = N * C * 4 + N * C * 2
        report("qk_normed_prepare (bias, norm of the whole of q and of k, rotation)",
               lambda: ops.qk_normed_prepare(y, qw, kw, 1e-6, freq[:d // 4], "half", 1.0, positions, seq, bt, qo, pages, G, d, P, bias=bias, whole=True), nbytes)
        report("qk_normed_prepare (no norm, rotation of the whole head)",
               lambda: ops.qk_normed_prepare(y, None, None, 1e-6, freq, "half", 1.0, positions, seq, bt, qo, pages, G, d, P), nbytes)
        report("  Tomodra: qk_normed_prepare (norm per head, neighbouring pairs)",
               lambda: ops.qk_normed_prepare(y, qw[:d].contiguous(), kw[:d].contiguous(), 1e-6, freq[:d // 4], "neighbours", 1.0, positions, seq, bt, qo, pages, G, d, P), nbytes)
        # ---- the gate on the heads' outputs, beside the gate per head
        out = torch.randn(N, H, d, device=dev).to(bf)
        gate_h = torch.rand(N, H, device=dev)
        report("sigmoid_gate (a logit per output element)", lambda: ops.sigmoid_gate(out.view(N, H * d), proj[:, C:], seq), N * H * d * 8)
        report("  Bivizen: head_gate (a gate per head)", lambda: ops.head_gate(out, gate_h, seq), N * H * d * 4)
        if label == "prompt":
            # ---- a prompt's attention on the tcgen05 kernel with the cap and the sink, beside the dense decoder's
            from air_b200.parts.attention import TiledAttention
            from air_b200.parts.base import HostBatch
            planner = type("P", (TiledAttention,), {"heads": H, "window": None})()
            plan = planner.plan(HostBatch(counts=[T], lengths=[0], slots=[0], q_start=[0, T]))
            tiles_ = i32(plan.arrays["tiles"].tolist())
            p5, ao, sk = pages.view(-1, 2, G, P, d), torch.empty(N, H, d, dtype=bf, device=dev), torch.randn(H, device=dev)
            fl = 4 * H * d * (T * (T + 1) // 2)
            report("prefill_attention_tc with a soft cap and learned sinks",
                   lambda: ops.prefill_attention_tc(qo, p5, bt, tiles_, ao, None, d ** -0.5, softcap=50.0, sink=sk), flops=fl)
            report("prefill_attention_tc with a zero sink",
                   lambda: ops.prefill_attention_tc(qo, p5, bt, tiles_, ao, None, d ** -0.5, sink=torch.zeros_like(sk)), flops=fl)
            report("  Qwen2: prefill_attention_tc", lambda: ops.prefill_attention_tc(qo, p5, bt, tiles_, ao, None, d ** -0.5), flops=fl)
        if label == "decode":
            # ---- single tokens over the pages: cap and sink, and the gate in the merge, beside Tomodra's chunk and sink
            sink = torch.randn(H, device=dev)
            ao = torch.empty(N, H, d, dtype=bf, device=dev)
            kvb = 2 * S * context * G * d * 2
            report("grouped_attention (all keys, soft cap, learned sink)",
                   lambda: ops.grouped_attention(qo, pages, bt, seq, positions, ao, None, d ** -0.5, kv_heads=G, page_tokens=P, sink=sink, softcap=50.0), kvb)
            report("grouped_attention (all keys, zero sink, gates in the merge)",
                   lambda: ops.grouped_attention(qo, pages, bt, seq, positions, ao, None, d ** -0.5, kv_heads=G, page_tokens=P, sink=torch.zeros_like(sink), gate=proj[:, C:]), kvb)
            p5 = pages.view(-1, 2, G, P, d)
            report("decode_attention (copy engine; soft cap, learned sink in the merge)",
                   lambda: ops.decode_attention(qo, p5, bt, seq, positions, ao, None, d ** -0.5, softcap=50.0, sink=sink), kvb)
            report("decode_attention (copy engine; zero sink and gates in the merge)",
                   lambda: ops.decode_attention(qo, p5, bt, seq, positions, ao, None, d ** -0.5, sink=torch.zeros_like(sink), gate=proj[:, C:]), kvb)
            report("  Qwen2: decode_attention (copy engine)",
                   lambda: ops.decode_attention(qo, p5, bt, seq, positions, ao, None, d ** -0.5), kvb)
            report("  Tomodra: grouped_attention (chunk of 1,024, sink)",
                   lambda: ops.grouped_attention(qo, pages, bt, seq, positions - 1, ao, None, d ** -0.5, kv_heads=G, page_tokens=P, chunk=1024, sink=sink), kvb // 2)
        # ---- retention beside gated linear attention (the same scan with a decay per channel)
        rq = torch.randn(N, 3 * H * d, device=dev)
        state = torch.zeros(S, H, d, d, device=dev)
        o = torch.empty(N, H, d, device=dev)
        decays, dec = torch.full((H,), 0.99, device=dev), torch.randn(N, H * d, device=dev)
        sb = (2 * S * H * d * d * 4 + N * 4 * H * d * 4) if label == "decode" else N * 4 * H * d * 4
        report("linear_scan as retention (rotation, a constant decay per head)",
               lambda: ops.linear_scan(ops.SCAN_RETENTION, rq[:, :H * d], rq[:, H * d:2 * H * d], rq[:, 2 * H * d:], decays, state, o, q_start, slots, seq, positions=positions, freq=freq, k_scale=d ** -0.5), sb)
        report("  Bivizen: linear_scan as gated linear attention",
               lambda: ops.linear_scan(ops.SCAN_GLA, rq[:, :H * d], rq[:, H * d:2 * H * d], rq[:, 2 * H * d:], dec, state, o, q_start, slots, seq, q_scale=d ** -0.5, tau=16.0), sb + N * H * d * 4)
        ones = torch.ones(d, device=dev)
        yo = torch.empty(N, H * d, dtype=bf, device=dev)
        report("gated_rmsnorm (norm per head without a weight's effect, silu gate)", lambda: ops.gated_rmsnorm(o, proj[:, :H * d], ones, 1e-6, yo, seq), N * H * d * 10)
        # ---- the squared rectifier, beside SiLU(gate) x up
        Fd = 3 * ff // 2
        z = torch.randn(N, Fd, device=dev).to(bf)
        zz = torch.randn(N, 2 * ff, device=dev).to(bf)
        act, act2 = torch.empty(N, Fd, dtype=bf, device=dev), torch.empty(N, ff, dtype=bf, device=dev)
        report("relu2 (behind the library's product)", lambda: ops.relu2(z, act), N * Fd * 4)
        report("  Qwen2: silu_mul", lambda: ops.silu_mul(zz, act2, block=128), N * ff * 6)
        xin = torch.randn(N, E, device=dev).to(bf)
        wup = torch.randn(Fd, E, device=dev).to(bf) * 0.02
        wgu = torch.randn(2 * ff, E, device=dev).to(bf) * 0.02
        if N <= 64 or N >= 512:
            bn = 256 if N <= 64 else 128
            report("gemm_tc with the squared rectifier in its epilogue (up)",
                   lambda: ops.gemm_tc(xin, wup, act, 256 if N <= 64 else 128, ops.EPI_RELU2), flops=2 * N * Fd * E) if N > 64 else \
                report("gemm_tc with the squared rectifier in its epilogue (up)",
                       lambda: ops.gemm_tc(xin, wup, act, 256, ops.EPI_RELU2), nbytes=Fd * E * 2)
            if N > 64:
                report("  Qwen2: gemm_tc with SiLU(gate) x up in its epilogue", lambda: ops.gemm_tc(xin, wgu, act2, 256, ops.EPI_SILU), flops=4 * N * ff * E)
            else:
                report("  Qwen2: gemm_tc with SiLU(gate) x up in its epilogue", lambda: ops.gemm_tc(xin, wgu, act2, 256, ops.EPI_SILU), nbytes=2 * ff * E * 2)
        # ---- the router with corrections and identity experts, the experts' two products
        total = n_exp + ident
        zr = torch.randn(N, 24, device=dev)
        corr = torch.randn(total, device=dev) * 0.1
        expert = torch.empty(N, top, dtype=torch.int32, device=dev)
        weight = torch.empty(N, top, device=dev)
        report("moe_route (softmax, score + correction, 18 outputs, top 4)", lambda: ops.moe_route(zr, total, top, expert, weight, score="softmax", choice_bias=corr), N * 24 * 4)
        e2, w2 = torch.empty(N, 2, dtype=torch.int32, device=dev), torch.empty(N, 2, device=dev)
        report("  Tomodra: moe_route (sigmoid, 16 experts, top 2)", lambda: ops.moe_route(zr, 16, 2, e2, w2, score="sigmoid"), N * 24 * 4)
        ops.moe_route(zr, total, top, expert, weight, score="softmax", choice_bias=corr)
        yp = torch.zeros(top, N, E, device=dev)
        report("moe_identity (the pairs of the two identity experts)", lambda: ops.moe_identity(xin, expert, weight, n_exp, yp), N * top * 2 // total * E * 6)
        pairs = N * top
        ints = torch.empty(n_exp + 1 + pairs + 2 * (pairs // ops.GROUP_TILE + n_exp) + 1, dtype=torch.int32, device=dev)
        start, pair_of_slot = ints[:n_exp + 1], ints[n_exp + 1:n_exp + 1 + pairs]
        tiles, num_tiles = ints[n_exp + 1 + pairs:-1].view(-1, 2), ints[-1:]
        ops.moe_sort(expert, n_exp, start, pair_of_slot, tiles, num_tiles)
        torch.cuda.synchronize()
        real = int(start[-1].item())
        touched = len(set(expert.view(-1).tolist()) - set(range(n_exp, total)))
        up = torch.randn(n_exp, F, E, device=dev).to(bf) * 0.02
        down = torch.randn(n_exp, E, F, device=dev).to(bf) * 0.02
        acts = torch.empty(pairs, F, dtype=bf, device=dev)
        if label == "decode":
            report("grouped_gemm up with the squared rectifier (few rows per expert)",
                   lambda: ops.grouped_gemm(xin, up, acts, F, E, lda=E, ldo=F, groups=n_exp, a_index=pair_of_slot, a_div=top, start=start, tiles=tiles, num_tiles=num_tiles, relu2=True),
                   nbytes=touched * F * E * 2)
            report("grouped_gemm down with the weight on the output",
                   lambda: ops.grouped_gemm(acts, down, yp, E, F, lda=F, ldo=E, groups=n_exp, o_index=pair_of_slot, o_div=top, o_part_stride=N * E, start=start, tiles=tiles, num_tiles=num_tiles, o_scale=weight.view(-1)),
                   nbytes=touched * F * E * 2)
        else:
            ends = start[1:].clone()
            rws = ops.rows_by_index(xin, pair_of_slot, top, None, torch.empty(pairs, E, dtype=bf, device=dev))
            report("library grouped product up + relu2 (many rows per expert)",
                   lambda: ops.relu2(torch._grouped_mm(rws, up.transpose(1, 2), offs=ends), acts), flops=2 * real * F * E)
            report("library grouped product down + planes_by_index with the weight",
                   lambda: ops.planes_by_index(torch._grouped_mm(acts, down.transpose(1, 2), offs=ends), pair_of_slot, top, yp, scale=weight.view(-1)),
                   flops=2 * real * F * E)
    return rows


def design_bench(args):
    import torch
    from air_b200.engine.batch import Entry, LAST_SAMPLED
    designs = {"bivizen": ("Bivizen", _bivizen), "tomodra": ("Tomodra", _tomodra), "pefivik": ("Pefivik", _pefivik),
               "tabopel": ("Tabopel", _tabopel)}
    # the model that stands beside the design: the Qwen2 decoder, or the closest of the other designs
    beside = {"pefivik": ("tomodra", "Tomodra", _tomodra), "tabopel": ("tomodra", "Tomodra", _tomodra)} \
        .get(args.design, ("qwen2", "Qwen2ForCausalLM", _qwen))
    if args.design not in designs:
        print(json.dumps({"error": f"--design {args.design}: the designs that are compared are {', '.join(designs)}"}))
        return 2
    title, make = designs[args.design]
    record = {"design": title, "beside": beside[1], "dtype": "bf16", "data": "synthetic", "sizes": {}}
    context = args.context or 2048
    for name in (args.design_sizes.split(",") if args.design_sizes else DESIGN_SIZES):
        width, layers, heads, kv_heads, ff = DESIGN_SIZES[name]
        if args.layers:
            layers = args.layers
        size = {"width": width, "layers": layers, "heads": heads, "kv_heads": kv_heads, "ff": ff}
        for label, cfg in ((args.design, make(width, layers, heads, kv_heads, ff)), (beside[0], beside[2](width, layers, heads, kv_heads, ff))):
            print(f"--- {label} at width {width}, {layers} layers", flush=True)
            size[label] = design_model(cfg, args, torch, Entry, LAST_SAMPLED)
        if not args.skip_kernels and args.design == "bivizen":
            size["kernels"] = design_kernels(width, heads, kv_heads, ff, args.prefill_tokens, args.batch, context)
        if not args.skip_kernels and args.design == "pefivik":
            size["kernels"] = pefivik_kernels(width, heads, kv_heads, ff, args.prefill_tokens, args.batch, context)
        if not args.skip_kernels and args.design == "tabopel":
            size["kernels"] = tabopel_kernels(width, heads, kv_heads, ff, args.prefill_tokens, args.batch, context)
        if not args.skip_kernels and args.design == "tomodra":
            size["kernels"] = tomodra_kernels(width, heads, kv_heads, ff, args.prefill_tokens, args.batch, context)
        record["sizes"][name] = size
    text = json.dumps(record)
    print(text)
    if args.output:
        with open(args.output, "w") as f:
            f.write(text + "\n")
    return 0


def reference_arm(args, cfg, context):
    """EmersonDowell/AIR's CUDA executor on the same shape: its own prefill and step_greedy_batch."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm as ref
    try:
        if args.batch > 8:
            raise ref.Unavailable("AIR decodes at most 8 sequences together (kMaxNativeDecodeBatch)")
        ref.build()
        clocks = ClockSampler()
        r = ref.bench(layers=args.layers or cfg["num_hidden_layers"], hidden=cfg["hidden_size"],
                      ffn=cfg["intermediate_size"], heads=cfg["num_attention_heads"],
                      kv_heads=cfg["num_key_value_heads"], vocab=cfg["vocab_size"],
                      max_positions=cfg["max_position_embeddings"], theta=cfg["rope_theta"], eps=cfg["rms_norm_eps"],
                      batch=args.batch, context=context, prefill=args.prefill_tokens, steps=args.steps,
                      warmup=args.warmup, fill="fork")
        clocks = clocks.stop()
    except ref.Unavailable as e:
        print(json.dumps({"impl": "reference", "unavailable": str(e)}))
        return 0
    ms = r["decode_ms_per_step"]
    value = args.batch / (ms / 1e3)
    line = {
        "metric": f"decode tok/s at batch {args.batch} (Qwen2.5-{args.shape.upper()} shape, bf16 weights, random weights)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "impl": "reference",
        "config": {"model": f"Qwen2.5-{args.shape.upper()} shape", "layers": args.layers or cfg["num_hidden_layers"],
                   "layers_of_model": cfg["num_hidden_layers"], "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": args.batch,
                   "seq_len": context, "context": context, "page_tokens": 16, "prefill_tokens": args.prefill_tokens,
                   "parallelism": "single GPU",
                   "same_config": "same shape, batch, context and bf16 weights; AIR keeps activations and cache in "
                                  "float32 and runs its own scalar kernels; the context is one computed prompt, "
                                  "forked (CudaKvCache::fork) for the other sequences",
                   "timing": "host clock around AIR's blocking calls (step_greedy_batch, prefill_greedy)"},
        # AIR's call takes host tokens and returns host tokens: it is end to end by construction
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 4 * args.batch,
                "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": None, "clocks": clocks,
        "prefill": {"value": r["prefill_tokens"] / (r["prefill_ms"] / 1e3) if r["prefill_ms"] > 0 else None,
                    "tokens": r["prefill_tokens"], "ms": r["prefill_ms"]},
        "reference_record": r,
    }
    print(json.dumps(line))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--shape", default="7b", help="7b, 14b, 32b, or a config.json of the architecture")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=0, help="tokens per request (default: 8192; 4096 at 32b)")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the shape has (for profiling)")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--repeats", type=int, default=5, help="timed repeats of K decode steps and of the prefill step")
    ap.add_argument("--prefill-pause-ms", type=float, default=200.0, help="idle time before every prefill repeat")
    ap.add_argument("--mixed", default="", help="D,P: also time one step of D decoding requests beside a P-token portion")
    ap.add_argument("--max-tokens", type=int, default=0, help="tokens in the cache pool (default: what device memory is left)")
    ap.add_argument("--output", default="", help="also write the JSON line to this file")
    ap.add_argument("--no-points", action="store_true", help="skip decoding at batch 1 and 64")
    ap.add_argument("--skip-prefill", action="store_true", help="for profiling the decode step alone")
    ap.add_argument("--skip-e2e", action="store_true", help="for profiling the decode step alone")
    ap.add_argument("--skip-decode", action="store_true", help="for profiling the prefill step alone")
    ap.add_argument("--no-graphs", action="store_true", help="launch the decode step's kernels one by one (for ncu)")
    ap.add_argument("--kernel", default="", help="prefill_attention, or prompt_elementwise (at --prefill-tokens rows): time those kernels alone and exit")
    ap.add_argument("--design", default="", help="bivizen, tomodra, pefivik or tabopel: prefill and decode of that design beside the Qwen2 decoder (pefivik and tabopel: beside Tomodra) at "
                    "equal sizes, and its kernels alone beside the like kernels (another line of output; the default "
                    "workload is not run)")
    ap.add_argument("--design-sizes", default="", help="with --design: which of the sizes 2048,4096 (default: both)")
    ap.add_argument("--skip-kernels", action="store_true", help="with --design: the models only")
    ap.add_argument("--timeline", action="store_true", help="also print the kernels' spans inside the decode graph and in the prefill step")
    args = ap.parse_args()
    if args.gpus != 1:
        print(json.dumps({"error": f"this engine runs on one GPU; --gpus {args.gpus} is not supported",
                          "n_gpus": args.gpus}))
        return 2
    args.warmup = max(args.warmup, 3)
    if args.design:
        return design_bench(args)
    if args.shape in SHAPES:
        cfg, context = dict(SHAPES[args.shape]), args.context or CONTEXTS[args.shape]
    else:
        with open(args.shape) as f:
            cfg = json.load(f)
        context = args.context or 8192
        args.shape = os.path.splitext(os.path.basename(args.shape))[0]
    if args.impl == "reference":
        return reference_arm(args, cfg, context)
    if args.kernel:
        if args.kernel == "prompt_elementwise":
            return kernel_prompt_elementwise(cfg, args.prefill_tokens)
        if args.kernel != "prefill_attention":
            print(json.dumps({"error": f"--kernel {args.kernel}: prefill_attention and prompt_elementwise are timed alone"}))
            return 2
        return kernel_prefill_attention(cfg)
    layers_of_model = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
        if "max_window_layers" in cfg:
            cfg["max_window_layers"] = args.layers

    import torch
    from air_b200.engine.batch import Entry, LAST_SAMPLED
    from air_b200.engine.engine import Engine, EngineConfig
    pk = peaks()
    mixed = tuple(int(x) for x in args.mixed.split(",")) if args.mixed else None
    batches = [args.batch] if args.no_points else sorted({1, args.batch, 64})
    most = max(batches + ([mixed[0] + 1] if mixed else []))
    page = 64
    engine = Engine.from_random(cfg, seed=0, config=EngineConfig(
        dtype=torch.bfloat16, page_tokens=page, max_tokens=args.max_tokens or None, max_requests=most + 1,
        cuda_graphs=not args.no_graphs))
    mc = engine.model_config
    pool_tokens = engine.cache.num_pages * page
    per_request = -(-(context + 8) // page) * page
    batches = [b for b in batches if b * per_request <= pool_tokens] or [1]
    if args.batch not in batches:
        print(json.dumps({"error": f"the cache pool holds {pool_tokens} tokens: too few for batch {args.batch} at "
                                   f"{context} tokens"}))
        return 1
    weight_bytes = engine.model.weight_bytes()
    kv_bytes_per_token = engine.cache.bytes_per_page(engine.model.cache_needs(), page, torch.bfloat16) // page
    randomize_cache(engine, torch)

    results = {}
    if args.skip_decode:
        batches, args.skip_e2e = [], True
        results[args.batch] = {"times": [float("nan")], "ms": float("nan"), "clocks": None, "launches": 0}
    for b in batches:
        requests = [f"r{i}" for i in range(b)]
        times, clocks, launches = decode_device(engine, requests, context, args.steps, args.warmup,
                                                args.repeats if b == args.batch else max(1, min(3, args.repeats)),
                                                torch, Entry, LAST_SAMPLED)
        results[b] = {"times": times, "ms": statistics.median(times), "clocks": clocks, "launches": launches}
        if args.timeline and b == args.batch:
            decode_timeline(engine, requests, context, torch, Entry, LAST_SAMPLED)
        if b == args.batch and not args.skip_e2e:
            sec, h2d, d2h = decode_e2e(engine, requests, context, args.steps, args.warmup, torch)
            results[b]["e2e"] = {"value": b / sec, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                                 "d2h_bytes_per_step": d2h}

    # prefill of one request, one step
    T = args.prefill_tokens
    g = torch.Generator().manual_seed(7)
    prompt = torch.randint(0, mc.vocab_size, (T,), generator=g).tolist()
    times = []
    for i in range(0 if args.skip_prefill else 2 + max(1, args.repeats)):
        torch.cuda.synchronize()
        # A prompt's prefill is a burst of some tens of milliseconds, not a sustained load: every repeat starts
        # after a pause, so that it is not timed at the clocks that the repeats before it left (seven steps back
        # to back run into the power limit: 23.4, 23.4, 24.3, 25.0, 24.6 ms were measured so).
        time.sleep(args.prefill_pause_ms / 1e3)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        engine.step([Entry("p", prompt, [T - 1])])
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
        engine.finish("p")
    pre_ms = statistics.median(times[2:]) if times else float("nan")       # (the first two steps are warm-up)
    if args.timeline and not args.skip_prefill:
        prefill_timeline(engine, prompt, torch, Entry)
    L, E, I, V = len(engine.model.spec.order), mc.hidden_size, mc.intermediate_size, mc.vocab_size
    H, K, d = mc.num_attention_heads, mc.num_key_value_heads, mc.head_dim
    gemm_params = L * (E * (H + 2 * K) * d + H * d * E + 3 * E * I)
    flops = 2 * T * gemm_params + L * 4 * H * d * (T * (T + 1) // 2) + 2 * E * V
    prefill = {"value": T / (pre_ms / 1e3), "tokens": T, "ms": pre_ms, "repeat_ms": times[2:],
               "pause_ms": args.prefill_pause_ms,
               "frac": flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12)}
    if "bf16_tflops_sustained" in pk:      # the step is tens of milliseconds long: also against the figure under the power cap
        prefill["frac_sustained"] = flops / (pre_ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12)

    mixed_record = None
    if mixed:
        D, P = mixed
        dev_ms, host_ms, prior = mixed_step(engine, D, P, context, max(5, args.repeats), torch, Entry)
        live = (D * context + prior + P) * kv_bytes_per_token
        step_flops = 2 * (D + P) * gemm_params + L * 4 * H * d * (P * prior + P * (P + 1) // 2) + 2 * E * V * D
        # The step's kernels run one after the other: the decode attention is bound by the cache it reads, the
        # products and the portion's attention by their flops (or by the weights, if those take longer to read).
        cache_ms = D * context * kv_bytes_per_token / (pk["hbm_gbs"] * 1e9) * 1e3
        product_ms = max(2 * (D + P) * gemm_params / (pk["bf16_tflops"] * 1e12), weight_bytes / (pk["hbm_gbs"] * 1e9)) * 1e3
        attention_ms = L * 4 * H * d * (P * prior + P * (P + 1) // 2) / (pk["bf16_tflops"] * 1e12) * 1e3
        mixed_record = {"decode": D, "portion": P, "portion_prior_tokens": prior, "device_ms": dev_ms,
                        "host_ms": host_ms, "tokens_per_s": (D + P) / (dev_ms / 1e3),
                        "bytes_frac": (weight_bytes + live) / (dev_ms / 1e3) / 1e9 / pk["hbm_gbs"],
                        "flops_frac": step_flops / (dev_ms / 1e3) / (pk["bf16_tflops"] * 1e12),
                        "roofline_ms": cache_ms + product_ms + attention_ms,
                        "frac": (cache_ms + product_ms + attention_ms) / dev_ms}

    main_r = results[args.batch]
    ms = main_r["ms"]

    def bytes_a_second(batch):        # what a decode step at this batch has to read, over its time (GB/s)
        live = batch * (context - (args.steps + 2) // 2) * kv_bytes_per_token
        return (weight_bytes + live) / (results[batch]["ms"] / 1e3) / 1e9
    achieved = bytes_a_second(args.batch)
    line = {
        "metric": f"decode tok/s at batch {args.batch} (Qwen2.5-{args.shape.upper()} shape, bf16, random weights)",
        "value": args.batch / (ms / 1e3), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": f"Qwen2.5-{args.shape.upper()} shape", "layers": L, "layers_of_model": layers_of_model,
                   "hidden": E, "heads": H, "kv_heads": K, "head_dim": d, "intermediate": I, "vocab": V,
                   "global_batch": args.batch, "seq_len": context, "context": context,
                   "page_tokens": page, "pool_tokens": pool_tokens, "prefill_tokens": T, "repeats": args.repeats,
                   "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (weights read every step)", "peaks": pk["source"]},
        "repeat_ms_per_step": main_r["times"],
        "e2e": main_r.get("e2e"),
        "gpu_launches": main_r["launches"],
        "clocks": main_r["clocks"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"]},
        "points": {f"decode_b{b}": b / (results[b]["ms"] / 1e3) for b in batches if b != args.batch},
        "points_roofline_frac": {f"decode_b{b}": bytes_a_second(b) / pk["hbm_gbs"] for b in batches if b != args.batch},
    }
    if mixed_record:
        line["mixed"] = mixed_record
    text = json.dumps(line)
    print(text)
    if args.output:
        with open(args.output, "w") as f:
            f.write(text + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
