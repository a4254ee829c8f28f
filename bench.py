#!/usr/bin/env python3
"""Benchmark: decode tokens per second of the Qwen3-8B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]
    python bench.py --shape 32b            # the Qwen3-32B shape: batch 1/8/32 to context 8192
    python bench.py --workload serve       # continuous batching, the Qwen3-1.7B shape

Default run: the layer sizes of the Qwen3-8B shape with random weights in
bfloat16, a batch of 8 requests decoding at a context of 4096 tokens.  A "step"
is one decode step (one new token per request).  One JSON line is printed with

- ``value``: decoded tokens per second, timed on the device with CUDA events
  around exactly K steps after W warm-up steps (the step replays the engine's
  CUDA graph; token ids are fed from the host, nothing is read back);
- ``e2e``: the same through the Python entry point (``Engine.step``: scheduler,
  pinned host-to-device copy of the step's inputs, device sampling, read-back of
  the sampled ids each step);
- ``prefill``: one step over a 2,048-token prompt, with its fraction of the
  measured bf16 peak;
- ``roofline``: bytes the decode step must read (every weight once, the cache of
  the live requests) over its time, against the measured copy bandwidth;
- ``points``: decode tokens per second at batch 1 and 64, at batch 8 and 64 with
  64-token pages (the run itself has the reference's block size, 16 tokens), and the
  output tokens per second of the continuous-batching workload below;
- ``clocks``: SM clock and throttle reasons sampled during the timed region.

Between timed steps the inputs (15 GB of weights, gigabytes of cache) are far
larger than the 126 MB L2, so no explicit flush is needed.

``--workload serve``: 64 requests with prompts of 128 to 2048 tokens (uniform, seeded) and
256 output tokens each, all submitted at once to ``Engine.add_request`` and driven by
``Engine.step`` (scheduler, mixed steps of prompt portions beside decode tokens, admission
and page churn) on the Qwen3-1.7B shape: output and total tokens per second, mean time to
the first token, mean time between tokens, preemptions, and how the wall time splits
between the host inside ``Engine.step`` and the GPU.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=36,
    hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
    intermediate_size=12288, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
    tie_word_embeddings=False, max_position_embeddings=40960, hidden_act="silu",
    attention_bias=False, use_sliding_window=False)
QWEN3_1P7B = dict(QWEN3_8B, num_hidden_layers=28, hidden_size=2048, num_attention_heads=16,
                  num_key_value_heads=8, intermediate_size=6144, tie_word_embeddings=True)
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64,
                 num_key_value_heads=8, intermediate_size=25600)
# shape -> (config, name, context of the decode points, batches: the second is the headline)
SHAPES = {"8b": (QWEN3_8B, "Qwen3-8B", 4096, (1, 8, 64)),
          "1.7b": (QWEN3_1P7B, "Qwen3-1.7B", 4096, (1, 8, 64)),
          "32b": (QWEN3_32B, "Qwen3-32B", 8192, (1, 8, 32))}
CONTEXT = 4096
PREFILL_TOKENS = 2048
PAGE_SIZE = 16          # the reference's block size, and the configuration's


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 100 ms while running."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def mark(self):
        return len(self.rows)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()

    def summary(self, a=0, b=None):
        rows = self.rows[a:b] or self.rows
        sm = [float(r[0]) for r in rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names)
                   if any(len(r) > 3 + i and r[3 + i] == "Active" for r in rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(rows)}


def reference_arm():
    print(json.dumps({
        "impl": "reference",
        "unavailable": "bwasti/binfer is a Bun/TypeScript program (no setup.py or pyproject.toml: "
                       "pip reports 'not installable'); Bun is not installed and cannot be "
                       "installed offline, and its CMake build pins sm_90"}))
    return 0


def fill_cache(engine, runner, n_req, length, vocab, gen):
    """n_req live requests holding ``length`` tokens each, prefilled through the step function."""
    import torch
    from binfer_b200.engine.runner import StepItem
    rids = []
    for i in range(n_req):
        rid = f"bench{i}"
        runner.add_request(rid)
        toks = torch.randint(0, vocab, (length,), generator=gen).tolist()
        for a in range(0, length, 2048):
            runner.step([StepItem(rid, toks[a:a + 2048], [])])
        rids.append(rid)
    torch.cuda.synchronize()
    return rids


def time_decode(runner, sampler, rids, vocab, steps, warmup, gen, clocks=None):
    """Device time of ``steps`` decode steps (graph replay + greedy sampling)."""
    import torch
    from binfer_b200.csrc import ops
    from binfer_b200.engine.runner import StepItem
    from binfer_b200.sampling import SamplingParams
    B = len(rids)
    params = [SamplingParams(temperature=0.0, seed=0) for _ in rids]
    toks = torch.randint(0, vocab, (steps + warmup, B), generator=gen).tolist()

    def one(i):
        logits = runner.step([StepItem(r, [toks[i][b]], [0]) for b, r in enumerate(rids)])
        return sampler.sample_async(logits, params, [0] * B, [[]] * B)

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    a = clocks.mark() if clocks else 0
    l0 = ops.launches()
    g0 = getattr(runner, "graph_kernel_launches", 0)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(warmup, warmup + steps):
        one(i)
    end.record()
    torch.cuda.synchronize()
    b = clocks.mark() if clocks else 0
    ms = start.elapsed_time(end)
    launches = (ops.launches() - l0) + (getattr(runner, "graph_kernel_launches", 0) - g0)
    return ms / steps, launches, (a, b)


def serve_workload(engine, vocab, n_req=64, lo=128, hi=2048, n_out=256, seed=0):
    """64 requests at once through Engine.add_request / Engine.step; the measures of the
    reference's live loop (src/serve.ts:280-550): throughput, time to first token, time
    between tokens."""
    import torch
    from binfer_b200.sampling import SamplingParams
    gen = torch.Generator().manual_seed(seed)
    lens = torch.randint(lo, hi + 1, (n_req,), generator=gen).tolist()
    prompts = [torch.randint(0, vocab, (n,), generator=gen).tolist() for n in lens]
    engine.warm_up()
    engine.time_gpu, engine.gpu_spans, engine.step_ms = True, [], []
    pre0 = engine.scheduler.num_preemptions
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    rids = [engine.add_request(p, SamplingParams(max_tokens=n_out, ignore_eos=True, seed=i))
            for i, p in enumerate(prompts)]
    first, last, seen = {}, {}, {r: 0 for r in rids}
    steps = 0
    while engine.has_work():
        arrived = engine.step()
        now = time.perf_counter() - t0
        steps += 1
        for req in arrived:
            n = len(req.output) - req.unresolved
            if n > seen.get(req.rid, 0):
                first.setdefault(req.rid, now)
                last[req.rid] = now
                seen[req.rid] = n
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    engine.time_gpu = False
    gpu_ms = sum(a.elapsed_time(b) for a, b, _ in engine.gpu_spans)
    outs = [engine.requests.pop(r) for r in rids]
    n_out_total = sum(len(r.output) for r in outs)
    itl = [(last[r] - first[r]) / (seen[r] - 1) for r in rids if seen[r] > 1]
    return {
        "requests": n_req, "prompt_tokens": sum(lens), "output_tokens": n_out_total,
        "wall_s": wall, "output_tok_s": n_out_total / wall,
        "total_tok_s": (sum(lens) + n_out_total) / wall,
        "ttft_ms_mean": 1e3 * statistics.mean(first.values()),
        "ttft_ms_max": 1e3 * max(first.values()),
        "itl_ms_mean": 1e3 * statistics.mean(itl),
        "preemptions": engine.scheduler.num_preemptions - pre0, "steps": steps,
        "host_step_s": sum(engine.step_ms) / 1e3, "gpu_busy_s": gpu_ms / 1e3,
        "gpu_idle_frac": max(0.0, 1.0 - gpu_ms / 1e3 / wall),
    }


def serve_point(peaks, layers=None, page_size=PAGE_SIZE):
    """The continuous-batching workload on the Qwen3-1.7B shape, with the bound its decode
    steps have (every weight once and the live cache at the copy bandwidth, batch 64)."""
    import torch
    from binfer_b200 import Engine, Qwen3Config
    raw = dict(QWEN3_1P7B)
    full = raw["num_hidden_layers"]
    if layers:
        raw["num_hidden_layers"] = layers
    cfg = Qwen3Config.from_dict(raw)
    engine = Engine(cfg, "bfloat16", random_seed=1, page_size=page_size, max_seq_len=4096,
                    max_batch_size=64, max_tokens_per_step=2048,
                    num_pages=64 * (4096 // page_size) + 64)
    r = serve_workload(engine, cfg.vocab_size)
    weight_bytes = engine.model.weight_bytes()
    mean_ctx = r["prompt_tokens"] / r["requests"] + 128
    step_s = (weight_bytes + 64 * mean_ctx * cfg.kv_bytes_per_token(2)) / (peaks["hbm_gbs"] * 1e9)
    r["decode_bound_tok_s"] = 64 / step_s
    r["layers"], r["layers_of_full_config"] = cfg.num_hidden_layers, full
    engine.runner.check_errors()
    del engine
    torch.cuda.empty_cache()
    return r


def profile_steps(args):
    """Per-kernel time of one prefill step and of one decode step, eager (event pairs around
    every launch: short kernels read longer than inside a captured step, so shares, not
    sums, are what to read)."""
    import torch
    from binfer_b200 import Engine, Qwen3Config
    from binfer_b200.engine.runner import StepItem
    from binfer_b200.profiling import Profiler
    base, shape_name, context, batches = SHAPES[args.shape]
    raw = dict(base)
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    cfg = Qwen3Config.from_dict(raw)
    B = args.batch or batches[1]
    ps = args.page_size
    engine = Engine(cfg, "bfloat16", random_seed=0, num_pages=B * (context // ps) + 64 + 256,
                    page_size=ps, max_seq_len=context, max_batch_size=B + 1,
                    max_tokens_per_step=2048, cuda_graphs=False)
    runner = engine.runner
    gen = torch.Generator().manual_seed(0)
    toks = torch.randint(0, cfg.vocab_size, (PREFILL_TOKENS,), generator=gen).tolist()

    def prefill():
        runner.add_request("pf")
        runner.step([StepItem("pf", toks, [PREFILL_TOKENS - 1])])
        runner.free_request("pf")

    rids = fill_cache(engine, runner, B, context - 16, cfg.vocab_size, gen)
    decode_items = [StepItem(r, [7 + i], [0]) for i, r in enumerate(rids)]
    n = 3
    for name, fn in ((f"prefill of {PREFILL_TOKENS} tokens", prefill),
                     (f"decode step, batch {B}, context {context}", lambda: runner.step(decode_items))):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        prof = Profiler()
        for _ in range(n):
            fn()
        prof.stop()
        rows = sorted(prof.collect().items(), key=lambda kv: -kv[1][1])
        total = sum(ms for _, (_, ms) in rows)
        print(f"\n{shape_name} shape, {cfg.num_hidden_layers} layers: {name} "
              f"(mean of {n}, {total / n:.2f} ms of kernels)")
        for kernel, (calls, ms) in rows:
            print(f"  {kernel:<30}{calls // n:>6} calls{ms / n:>10.3f} ms{100 * ms / total:>7.1f} %")
    runner.check_errors()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES),
                    help="layer sizes: the headline's Qwen3-8B, or the 1.7B / 32B shapes")
    ap.add_argument("--workload", default="decode", choices=["decode", "serve"],
                    help="serve: the continuous-batching workload on the Qwen3-1.7B shape")
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--page-size", type=int, default=PAGE_SIZE)
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers than the configuration has (named in the record)")
    ap.add_argument("--no-points", action="store_true", help="skip the other batches, the "
                    "16-token pages, the serve workload and the prefill")
    ap.add_argument("--decode-only", action="store_true",
                    help="only the device-timed decode steps (for profiling): no e2e, no points")
    ap.add_argument("--eager", action="store_true", help="no CUDA graphs (for profiling)")
    ap.add_argument("--profile", action="store_true",
                    help="instead of the bench line: per-kernel CUDA events of a prefill of 2,048 "
                         "tokens and of a decode step at --batch (eager launches; the "
                         "reference's spans: src/profiler/profiler.ts:93-479)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    peaks = load_peaks()
    if args.profile:
        return profile_steps(args)
    if args.workload == "serve":
        r = serve_point(peaks, args.layers, args.page_size)
        print(json.dumps({"metric": "continuous batching, 64 requests x [128, 2048] prompt "
                                    "tokens x 256 output tokens (Qwen3-1.7B shape, bf16, 1 B200)",
                          "value": r["output_tok_s"], "unit": "output tokens/s", "n_gpus": 1,
                          "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
                          "impl": "ours", "serve": r}))
        return 0

    import torch
    from binfer_b200 import Engine, Qwen3Config
    from binfer_b200.csrc import ops
    from binfer_b200.engine import make_runner
    from binfer_b200.engine.runner import StepItem

    base, shape_name, context, batches = SHAPES[args.shape]
    raw = dict(base)
    full_layers = raw["num_hidden_layers"]
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    cfg = Qwen3Config.from_dict(raw)
    steps, warmup = args.steps, args.warmup
    B = args.batch or batches[1]
    page_size = args.page_size
    if args.decode_only:
        args.no_points = True
    max_b = max(B, 1 if args.no_points else max(batches))
    pages = max_b * (context // page_size) + 64
    t0 = time.time()
    engine = Engine(cfg, "bfloat16", random_seed=0, num_pages=pages, page_size=page_size,
                    max_seq_len=context, max_batch_size=max_b, max_tokens_per_step=2048,
                    cuda_graphs=not args.eager)
    runner, sampler = engine.runner, engine.sampler
    vocab = cfg.vocab_size
    gen = torch.Generator().manual_seed(0)
    load_s = time.time() - t0

    weight_bytes = engine.model.weight_bytes() - engine.model.embed.numel() * 2 * (
        0 if cfg.tie_word_embeddings else 1)
    kv_per_token = cfg.kv_bytes_per_token(2)

    clocks = ClockSampler()
    clocks.start()

    def decode_point(batch, n_steps, n_warm, run=None):
        run = run or runner
        start_len = context - (n_steps + n_warm)
        rids = fill_cache(engine, run, batch, start_len, vocab, gen)
        ms, launches, span = time_decode(run, sampler, rids, vocab, n_steps, n_warm, gen, clocks)
        mean_ctx = start_len + n_warm + n_steps / 2
        for r in rids:
            run.free_request(r)
        return ms, launches, span, mean_ctx

    def hbm_frac(batch, ms, mean_ctx):
        return (weight_bytes + batch * mean_ctx * kv_per_token) / (ms / 1e3) / 1e9 / peaks["hbm_gbs"]

    # ---- the headline: batch B at the shape's context
    ms_step, launches, span, mean_ctx = decode_point(B, steps, warmup)
    value = B / (ms_step / 1e3)
    bytes_step = weight_bytes + B * mean_ctx * kv_per_token
    achieved = bytes_step / (ms_step / 1e3) / 1e9
    clk = clocks.summary(*span)
    if clk["samples"] < 3:
        # a short timed region falls between two samples of the clock: time it once more,
        # long enough for a few of them (these steps are not the reported ones)
        extra = max(steps, int(600 / max(ms_step, 0.1)))
        _, _, span2, _ = decode_point(B, min(extra, context // 4), warmup)
        clk = clocks.summary(*span2)
        clk["note"] = "sampled over a longer run of the same steps"

    if args.decode_only:
        clocks.stop()
        print(json.dumps({"decode_only": True, "ms_per_step": ms_step, "value": value,
                          "layers": cfg.num_hidden_layers, "batch": B, "shape": args.shape,
                          "page_size": page_size,
                          "roofline_frac": achieved / peaks["hbm_gbs"], "clocks": clk}))
        return 0

    # ---- end to end through the entry point: scheduler, H2D inputs, D2H ids every step
    # (the clock sampler is stopped first: its nvidia-smi queries contend with the host's
    # CUDA calls, which this measurement, unlike the device-timed one, has in its loop)
    clocks.stop()
    # prompts are prefilled in portions, so the requests start decoding a few steps apart;
    # they are given room enough that none finishes (and the batch does not shrink) while
    # the steps are timed
    slack = 2 * B + 8
    prompts = [torch.randint(0, vocab, (context - (steps + warmup) - slack,),
                             generator=gen).tolist() for _ in range(B)]
    from binfer_b200.sampling import SamplingParams
    for p in prompts:
        engine.add_request(p, SamplingParams(max_tokens=steps + warmup + slack - 1,
                                             ignore_eos=True, seed=0))
    while any(r.remaining > 1 or not r.output for r in engine.scheduler.running) \
            or engine.scheduler.waiting:
        engine.step()                                   # prefill portions
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    h0, d0 = runner.h2d_bytes + sampler.h2d_bytes, sampler.d2h_bytes
    t1 = time.perf_counter()
    n_e2e = 0
    for _ in range(steps - 1):
        n_e2e += len(engine.step())
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t1
    e2e = {"value": n_e2e / e2e_s, "unit": "tokens/s",
           "h2d_bytes_per_step": (runner.h2d_bytes + sampler.h2d_bytes - h0) // max(steps - 1, 1),
           "d2h_bytes_per_step": (sampler.d2h_bytes - d0) // max(steps - 1, 1)}
    while engine.has_work():
        engine.step()

    points, fracs, prefill, serve = {}, {}, None, None
    if not args.no_points:
        for b in batches:
            if b == B:
                continue
            ms_b, _, _, ctx_b = decode_point(b, steps, warmup)
            points[f"decode_b{b}"] = b / (ms_b / 1e3)
            fracs[f"decode_b{b}"] = round(hbm_frac(b, ms_b, ctx_b), 4)
        # ---- prefill of 2,048 tokens in one step
        toks = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()
        times = []
        for i in range(5):
            runner.add_request("pf")
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            runner.step([StepItem("pf", toks, [PREFILL_TOKENS - 1])])
            e.record()
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e))
            runner.free_request("pf")
        pf_ms = statistics.median(times[2:])
        L, H, I = cfg.num_hidden_layers, cfg.hidden_size, cfg.intermediate_size
        Q, KV = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
        T = PREFILL_TOKENS
        flops = L * (2 * T * (H * (Q + 2 * KV) + Q * H + 3 * H * I)
                     + 4 * cfg.num_attention_heads * cfg.head_dim * T * (T + 1) / 2) \
            + 2 * H * vocab
        prefill = {"value": T / (pf_ms / 1e3), "tokens": T, "ms": pf_ms,
                   "frac": flops / (pf_ms / 1e3) / (peaks["bf16_tflops"] * 1e12)}
        if args.shape == "8b":
            # ---- the same model over a cache of the other page size (64 tokens, or 16)
            other = 64 if page_size != 64 else 16
            second = make_runner(engine.model, engine.env, page_size=other,
                                 num_pages=max(batches) * (context // other) + 64,
                                 max_requests=max(batches))
            second.enable_decode_graphs(max_batch=max(batches), max_seq_len=context)
            for b in (B, max(batches)):
                ms_b, _, _, ctx_b = decode_point(b, steps, warmup, run=second)
                points[f"decode_b{b}_page{other}"] = b / (ms_b / 1e3)
                fracs[f"decode_b{b}_page{other}"] = round(hbm_frac(b, ms_b, ctx_b), 4)
            second.check_errors()
            del second
    runner.check_errors()
    if not args.no_points and args.shape == "8b":
        del engine, runner
        torch.cuda.empty_cache()
        serve = serve_point(peaks)
        points["serve_1p7b_output_tok_s"] = serve["output_tok_s"]

    out = {
        "metric": f"decode tok/s @ batch {B}, context {context} ({shape_name} shape, bf16, 1 B200)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {
            "model": f"{shape_name} shape, random weights", "layers": cfg.num_hidden_layers,
            "layers_of_full_config": full_layers, "hidden": cfg.hidden_size,
            "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size,
            "vocab": cfg.vocab_size, "tied": cfg.tie_word_embeddings, "global_batch": B,
            "seq_len": context, "page_size": page_size, "parallelism": "1 GPU",
            "cuda_graphs": not args.eager, "l2": f"inputs larger than L2 (weights {weight_bytes / 1e9:.0f} GB per step)",
            "clocks_sampled": "during the device-timed steps",
            "peaks": peaks["source"],
        },
        "clocks": clk,
        "e2e": e2e,
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"]},
        "points": points,
        "points_hbm_frac": fracs,
    }
    if prefill is not None:
        out["prefill"] = prefill
    if serve is not None:
        out["serve"] = serve
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
