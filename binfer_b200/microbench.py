"""Time one of the engine's kernels alone, at a given size, against its roofline.

    python -m binfer_b200.microbench decode_attention --batch 8 --ctx 4096
    python -m binfer_b200.microbench prefill_attention --tokens 2048
    python -m binfer_b200.microbench gemm --tokens 8 --features 6144 --k 4096 [--library]
    python -m binfer_b200.microbench add_rmsnorm --tokens 8 --hidden 4096
    BINFER_B200_TRACE=1 python -m binfer_b200.microbench step_timeline --batch 8 --ctx 4096 --layers 6

Sizes default to the Qwen3-8B shape.  Each kernel runs on a rotation of input sets
larger than the L2 cache, after warm-up, between CUDA events; the line printed gives
microseconds per launch, the bytes or flops the kernel has to move, and the
fraction of the measured peak (``MEASURED_PEAKS.json`` beside the package, else the
stated fallback).  The reference measures its own peaks the same way at run time
(src/profiler/profiler.ts:553-659).  ``--iters 1 --warmup 0`` gives a run small
enough to put under a profiler.

``step_timeline`` runs whole decode steps of a random-weight model of the given layer sizes
(CUDA graphs, as in serving) with the library built for tracing (``BINFER_B200_TRACE=1``
must be set before the first import: the kernels of the step then record the GPU's global
timer when their first block starts, when its dependency wait returns and when it ends)
and prints the last step's events in order, with the time since the previous one.  Library
products are not instrumented; they show as the gaps around the engine's own kernels.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

from .csrc import ops

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BF16 = torch.bfloat16


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


GRAPH = True


def timed(fns, iters, warmup):
    """Microseconds per call of fns[i % len(fns)]() (a rotation of input sets).  The calls
    are captured into one CUDA graph, as the engine's decode step is, so that the host's
    launch cost does not hide the time of a short kernel."""
    for i in range(max(warmup, 1)):
        fns[i % len(fns)]()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if GRAPH and iters > 1:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(iters):
                fns[i % len(fns)]()
        g.replay()
        torch.cuda.synchronize()
        a.record()
        g.replay()
        b.record()
    else:
        a.record()
        for i in range(iters):
            fns[i % len(fns)]()
        b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / iters


def report(name, us, nbytes=None, flops=None, **extra):
    hbm, tf, src = peaks()
    out = {"kernel": name, "us": round(us, 2), **extra}
    if nbytes is not None:
        out["GB/s"] = round(nbytes / us / 1e3, 1)
        out["frac_of_hbm_peak"] = round(nbytes / us / 1e3 / hbm, 3)
    if flops is not None:
        out["TFLOP/s"] = round(flops / us / 1e6, 1)
        out["frac_of_bf16_peak"] = round(flops / us / 1e6 / tf, 3)
    out["peaks"] = src
    print(json.dumps(out), flush=True)


def _paged_cache(dev, n_req, ctx, nkv, d, ps, sets, scattered=False):
    """Random caches for n_req requests of ctx tokens.  Pages: the eight (128 / ps) of each
    128-key tile side by side in the pool, the tiles themselves in shuffled order, as the
    page pool hands them out; with ``scattered`` every page anywhere."""
    pages_per = -(-ctx // ps)
    run = max(1, 128 // ps)
    pages_per = -(-pages_per // run) * run
    total = n_req * pages_per + 1
    out = []
    for s in range(sets):
        kc = torch.randn(total, nkv, ps, d, device=dev, dtype=BF16)
        vc = torch.randn(total, nkv, ps, d, device=dev, dtype=BF16)
        if scattered:
            perm = (torch.randperm(total - 1, device=dev) + 1).to(torch.int32)
        else:
            runs = torch.randperm((total - 1) // run, device=dev).to(torch.int32)
            perm = (runs[:, None] * run + 1 + torch.arange(run, device=dev, dtype=torch.int32)
                    ).reshape(-1)
        bt = perm[: n_req * pages_per].view(n_req, pages_per).contiguous()
        out.append((kc, vc, bt))
    return out


def decode_attention(a):
    dev = torch.device("cuda:0")
    B, ctx, nh, nkv, d, ps = a.batch, a.ctx, a.heads, a.kv_heads, a.head_dim, a.page_size
    per_set = 2 * B * ctx * nkv * d * 2
    sets = max(2, int(3e8 // per_set) + 1)
    caches = _paged_cache(dev, B, ctx, nkv, d, ps, sets, a.scattered)
    q = torch.randn(B, nh * d, device=dev, dtype=BF16)
    out = torch.empty_like(q)
    sot = torch.arange(B, dtype=torch.int32, device=dev)
    pos = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
    err = ops.error_word(dev)
    fns = [lambda c=c: ops.decode_attention(q, c[0], c[1], None, B, sot, pos, c[2], out, nh, nkv, d,
                                            None, d ** -0.5, ctx, err, variant=a.variant)
           for c in caches]
    us = timed(fns, a.iters, a.warmup)
    report("decode_attention", us, nbytes=per_set, batch=B, ctx=ctx, heads=nh, kv_heads=nkv,
           head_dim=d, page_size=ps)


def prefill_attention(a):
    dev = torch.device("cuda:0")
    T, start, nh, nkv, d, ps = a.tokens, a.start, a.heads, a.kv_heads, a.head_dim, a.page_size
    ctx = start + T
    (kc, vc, bt), = _paged_cache(dev, 1, ctx, nkv, d, ps, 1, a.scattered)
    q = torch.randn(T, nh * d, device=dev, dtype=BF16)
    out = torch.empty_like(q)
    items = torch.tensor([[0, 0, T, start]], dtype=torch.int32, device=dev)
    err = ops.error_word(dev)
    fn = lambda: ops.prefill_attention(q, kc, vc, items, 1, T, bt, out, nh, nkv, d, None,
                                       d ** -0.5, err,
                                       variant=a.variant if a.variant in ("umma2", "umma", "mma_sync")
                                       else "auto", max_ctx=ctx if a.splits < 0 else 0,
                                       splits=max(a.splits, 0))
    us = timed([fn], a.iters, a.warmup)
    flops = 4.0 * nh * d * (T * start + T * (T + 1) / 2)
    report("prefill_attention", us, flops=flops, tokens=T, start=start, heads=nh, kv_heads=nkv,
           head_dim=d)


def gemm(a):
    dev = torch.device("cuda:0")
    M, N, K = a.tokens, a.features, a.k
    sets = max(2, int(3e8 // (N * K * 2)) + 1)
    ws = [(0.05 * torch.randn(N, K, device=dev)).to(BF16) for _ in range(sets)]
    x = torch.randn(M, K, device=dev).to(BF16)
    out = torch.empty(M, N, device=dev, dtype=BF16)
    err = ops.error_word(dev)
    name = "gemm_bf16_tcgen05"
    if a.library:
        name = "gemm_library"
        fns = [lambda w=w: torch.mm(x, w.t(), out=out) for w in ws]
    elif a.pair:
        name = f"gemm_bf16_pair(bn={a.bn})"
        fns = [lambda w=w: ops.gemm_bf16_pair(x, w, out, err, a.bn) for w in ws]
    elif a.cluster:
        name = f"gemm_bf16_cluster(bn={a.bn},cluster={a.cluster})"
        fns = [lambda w=w: ops.gemm_bf16_cluster(x, w, out, err, a.bn, a.cluster) for w in ws]
    else:
        fns = [lambda w=w: ops.gemm_bf16(x, w, out, err, bn=a.bn) for w in ws]
    us = timed(fns, a.iters, a.warmup)
    report(name, us,
           nbytes=(N * K + M * K + M * N) * 2, flops=2.0 * M * N * K, tokens=M, features=N, k=K)


def swiglu(a):
    """The gate/up projection with the activation in its epilogue (--tokens, --intermediate,
    --k); --library times the library's product followed by the activation kernel."""
    dev = torch.device("cuda:0")
    M, I, K = a.tokens, a.intermediate, a.k
    sets = max(2, int(3e8 // (2 * I * K * 2)) + 1)
    ws = [(0.05 * torch.randn(2 * I, K, device=dev)).to(BF16) for _ in range(sets)]
    x = torch.randn(M, K, device=dev).to(BF16)
    out = torch.empty(M, I, device=dev, dtype=BF16)
    gu = torch.empty(M, 2 * I, device=dev, dtype=BF16)
    err = ops.error_word(dev)
    if a.library:
        name = "library product + silu_mul"

        def two(w):
            torch.mm(x, w.t(), out=gu)
            ops.silu_mul(gu, out)
        fns = [lambda w=w: two(w) for w in ws]
    elif a.pair:
        name = f"gemm_bf16_pair(gated,bn={a.bn})"
        fns = [lambda w=w: ops.gemm_bf16_pair(x, w, out, err, a.bn, gated=True) for w in ws]
    else:
        bn = a.bn or ops.gemm_swiglu_plan(I, K, dev)[0]
        name = f"gemm_bf16_swiglu(bn={bn})"
        fns = [lambda w=w: ops.gemm_bf16_swiglu(x, w, out, err, bn) for w in ws]
    us = timed(fns, a.iters, a.warmup)
    report(name, us, nbytes=(2 * I * K + M * K + M * I) * 2, flops=4.0 * M * I * K, tokens=M,
           intermediate=I, k=K)


def add_rmsnorm(a):
    dev = torch.device("cuda:0")
    T, H = a.tokens, a.hidden
    resid = torch.randn(T, H, device=dev)
    delta = torch.randn(T, H, device=dev).to(BF16)
    w = torch.ones(H, device=dev)
    out = torch.empty(T, H, device=dev, dtype=BF16)
    us = timed([lambda: ops.add_rmsnorm(resid, delta, w, out, 1e-6)], a.iters, a.warmup)
    report("add_rmsnorm", us, nbytes=T * H * (4 + 4 + 2 + 2), tokens=T, hidden=H)


def step_timeline(a):
    import ctypes
    from . import Engine
    from .config import Qwen3Config
    from .engine.runner import StepItem
    from .sampling import SamplingParams
    from .csrc import build
    if not build.TRACE:
        raise SystemExit("step_timeline: set BINFER_B200_TRACE=1 in the environment")
    dev = torch.device("cuda:0")
    B, ctx = a.batch, a.ctx
    raw = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=a.layers,
               hidden_size=a.hidden, num_attention_heads=a.heads, num_key_value_heads=a.kv_heads,
               head_dim=a.head_dim, intermediate_size=a.intermediate, vocab_size=a.vocab,
               rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False,
               max_position_embeddings=max(ctx, 4096), hidden_act="silu", attention_bias=False,
               use_sliding_window=False)
    cfg = Qwen3Config.from_dict(raw)
    ps = a.page_size
    eng = Engine(cfg, "bfloat16", random_seed=0, num_pages=B * (-(-ctx // ps)) + 64, page_size=ps,
                 max_seq_len=ctx, max_batch_size=B, max_tokens_per_step=2048, cuda_graphs=True)
    runner, sampler = eng.runner, eng.sampler
    gen = torch.Generator().manual_seed(0)
    steps = 8
    rids = []
    for i in range(B):
        rid = f"t{i}"
        runner.add_request(rid)
        toks = torch.randint(0, cfg.vocab_size, (ctx - steps - 1,), generator=gen).tolist()
        for s0 in range(0, len(toks), 2048):
            runner.step([StepItem(rid, toks[s0:s0 + 2048], [])])
        rids.append(rid)
    params = [SamplingParams(temperature=0.0, seed=0) for _ in rids]
    torch.cuda.synchronize()
    readers = [getattr(ops.lib(), "bf_trace_read_" + f) for f in
               ("elementwise", "qkv_post", "attention_decode_persistent", "attention_decode",
                "gemm_tcgen05_cluster")]
    times = (ctypes.c_ulonglong * 8192)()
    codes = (ctypes.c_int * 8192)()
    events = []
    for i in range(steps):
        if i == steps - 1:
            torch.cuda.synchronize()
            for rd in readers:
                rd(times, codes)                         # empty the lists: only the last step stays
        logits = runner.step([StepItem(r, [int(torch.randint(0, cfg.vocab_size, (1,), generator=gen))],
                                       [0]) for r in rids])
        sampler.sample_async(logits, params, [0] * B, [[]] * B)
    torch.cuda.synchronize()
    for rd in readers:
        n = rd(times, codes)
        events += [(times[i], codes[i]) for i in range(n)]
    events.sort()
    names = {1: "add_rmsnorm", 2: "silu_mul", 3: "qk_norm_rope", 4: "decode_attention",
             5: "attention_merge", 6: "gemm_cluster"}
    phases = ["first block starts", "wait returns", "ends", "partial sums sent",
              "cluster barrier passed", "products done"]
    t0 = prev = events[0][0]
    print(f"# decode step, batch {B}, context {ctx}, {a.layers} layers; microseconds", flush=True)
    for t, c in events:
        print(f"{(t - t0) / 1e3:10.2f} {(t - prev) / 1e3:8.2f}  {names.get(c // 10, '?'):18s} "
              f"{phases[c % 10]}  [{c}]")
        prev = t
    print(json.dumps({"kernel": "step_timeline", "us": round((events[-1][0] - t0) / 1e3, 2),
                      "events": len(events), "batch": B, "ctx": ctx, "layers": a.layers}))


def main(argv=None):
    ap = argparse.ArgumentParser(prog="python -m binfer_b200.microbench", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("kernel", choices=["decode_attention", "prefill_attention", "gemm",
                                       "swiglu", "add_rmsnorm", "step_timeline"])
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=8)
    ap.add_argument("--start", type=int, default=0, help="tokens already cached (prefill)")
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--scattered", action="store_true",
                    help="decode_attention: no two pages of a tile side by side in the pool")
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=6, help="step_timeline: layers of the model")
    ap.add_argument("--intermediate", type=int, default=12288)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--features", type=int, default=6144)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--bn", type=int, default=0, help="feature rows per tile (0: chosen)")
    ap.add_argument("--library", action="store_true", help="time cuBLAS on the same product")
    ap.add_argument("--splits", type=int, default=-1,
                    help="prefill attention: shares of the keys per block of 256 queries "
                         "(-1: chosen from the context, 1: none)")
    ap.add_argument("--pair", action="store_true",
                    help="gemm, swiglu: the kernel on pairs of SMs (many token rows)")
    ap.add_argument("--cluster", type=int, default=0,
                    help="gemm: split K over clusters of this many CTAs (needs --bn)")
    ap.add_argument("--no-graph", action="store_true", help="launch from the host, no CUDA graph")
    ap.add_argument("--variant", default="auto", choices=["auto", "persistent", "tma", "cp_async", "umma2", "umma", "mma_sync"],
                    help="decode attention: tma or cp_async tile loads; prefill attention: "
                         "umma (tcgen05) or mma_sync")
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("microbench needs a CUDA device", file=sys.stderr)
        return 1
    ops.lib()
    global GRAPH
    GRAPH = not a.no_graph
    {"decode_attention": decode_attention, "prefill_attention": prefill_attention,
     "gemm": gemm, "swiglu": swiglu, "add_rmsnorm": add_rmsnorm,
     "step_timeline": step_timeline}[a.kernel](a)
    return 0


if __name__ == "__main__":
    sys.exit(main())
