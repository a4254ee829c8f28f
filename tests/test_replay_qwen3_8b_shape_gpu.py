"""Replay at the real layer sizes of the Qwen3-8B shape (two layers of it) against the
plain implementation.

The tiny configurations never reach the kernels that a step of the full model runs: the
split-K cluster products for 6144x4096, 4096x4096 and 4096x12288 weights, the gate/up
product with the activation at 12288 inner features, the persistent decode attention at
32/8 heads, the tcgen05 prefill attention, the tcgen05 head product over 151936 words and
the captured decode step with block tables for long contexts.  Here they run as one model:
hidden 4096, 32 query and 8 kv heads of 128, 12288 inner features, an untied head over
151936 words, fewer layers (2 of 36).  What one layer does:
src/engine/batched_engine.ts:800-1314; final norm and head: :1733-1770.

Weights are stored in bfloat16; the float32 engine widens them (exact), and the plain
implementation reads the same stored values in float64.  Logits are compared at a
subset of positions (every fifth, the edges of 16- and 64-token pages, the last 40 of
each request), so that the comparison stays in memory.

Bounds.  float32: those of the tiny configurations.  bfloat16: the largest error is held
to the tiny configurations' bound; the root-mean-square error, which at this width is all
rounding (sums of 4096 and 12288 bfloat16 products, layer upon layer), is held to what the
reference's own arithmetic gives on the same tokens: the plain implementation with every
result rounded to bfloat16 where the reference stores it in bfloat16 (``round_to``).  The
engine keeps the residual stream, the norms' inputs and the logits in float32, so it has
to be at least as close to the exact result as that model is.
"""
import pytest
import torch

import helpers as H
import qwen3_plain as P
from test_replay_gpu import TOL, TOL_RMS, _Names

pytestmark = pytest.mark.gpu

LENGTHS = [1040, 70, 45, 130]
EXTRA = [55, 61]                      # join the mixed trace
VOCAB = H.QWEN3_8B_TWO_LAYERS["vocab_size"]
GRAPH_SEQ_LEN = 1280


def _requests(extra=False):
    lens = LENGTHS + (EXTRA if extra else [])
    return {f"r{i}": H.random_tokens(n, VOCAB, 100 * i + n) for i, n in enumerate(lens)}


def _keep(reqs):
    def keep(rid, p):
        return (p % 5 == 0 or p % 64 in (0, 15, 16, 63) or p >= len(reqs[rid]) - 40)
    return keep


class _Shape:
    """The model folder, its weights in float64 and the plain logits, each computed once."""

    def __init__(self, tmp):
        from binfer_b200.config import Qwen3Config
        from binfer_b200.weights import write_model_dir
        cfg = Qwen3Config.from_dict(H.QWEN3_8B_TWO_LAYERS)
        self.dir = write_model_dir(cfg, str(tmp / "qwen3_8b_two_layers"), seed=8, std=0.02,
                                   norm_std=0.05, dtype=torch.bfloat16)
        self.raw, w = H.read_model_dir(self.dir)
        self.w64 = {k: t.to(torch.float64) for k, t in w.items()}
        self.models = {}
        self.logits = {}
        self.rounded = {}

    def model(self, dtype):
        from binfer_b200.engine import make_env, model_from_dir
        if dtype not in self.models:
            env = make_env(dtype)
            self.models[dtype] = (model_from_dir(self.dir, env), env)
        return self.models[dtype]

    def runner(self, dtype, page_size, num_pages, graphs=False, max_requests=8):
        from binfer_b200.engine import make_runner
        model, env = self.model(dtype)
        r = make_runner(model, env, page_size=page_size, num_pages=num_pages,
                        max_requests=max_requests)
        if graphs:
            r.enable_decode_graphs(max_batch=8, max_seq_len=GRAPH_SEQ_LEN)
        return r

    def plain(self, reqs):
        """{request: {position: float64 logits}} at the kept positions."""
        keep = _keep(reqs)
        out = {}
        for rid, toks in reqs.items():
            key = (rid, tuple(toks))
            if key not in self.logits:
                rows = [p for p in range(len(toks)) if keep(rid, p)]
                lg = P.forward(self.raw, self.w64, toks, dtype=torch.float64, rows=rows)
                self.logits[key] = {p: lg[i] for i, p in enumerate(rows)}
            out[rid] = self.logits[key]
        return out


    def reference_rounding_rms(self, reqs):
        """Root-mean-square error, over the kept positions of ``reqs``, of the plain
        implementation rounding to bfloat16 wherever the reference does, against the exact
        one, relative to the exact logits' root mean square."""
        keep = _keep(reqs)
        exact = self.plain(reqs)
        num = den = 0.0
        for rid, toks in reqs.items():
            key = (rid, tuple(toks))
            if key not in self.rounded:
                rows = [p for p in range(len(toks)) if keep(rid, p)]
                lg = P.forward(self.raw, self.w64, toks, dtype=torch.float64, rows=rows,
                               round_to=torch.bfloat16)
                ex = torch.stack([exact[rid][p] for p in rows])
                self.rounded[key] = (float((lg - ex).pow(2).sum()), float(ex.pow(2).sum()))
            num += self.rounded[key][0]
            den += self.rounded[key][1]
        return (num / den) ** 0.5


@pytest.fixture(scope="module")
def shape(tmp_path_factory, cuda_device):
    s = _Shape(tmp_path_factory.mktemp("shape8b"))
    yield s
    s.models.clear()
    s.logits.clear()
    s.rounded.clear()
    s.w64.clear()
    torch.cuda.empty_cache()


def _compare(got, ref, dtype, what, rms_bound=None):
    assert got, "the trace produced no logits"
    worst, worst_at = 0.0, None
    for (rid, pos), row in got.items():
        e = H.rel_err(row, ref[rid][pos])
        if e > worst:
            worst, worst_at = e, (rid, pos)
    assert worst <= TOL[dtype], f"{what}: worst relative error {worst:.3g} at {worst_at}"
    num = sum(float((row.double() - ref[rid][pos]).pow(2).sum()) for (rid, pos), row in got.items())
    den = sum(float(ref[rid][pos].pow(2).sum()) for (rid, pos) in got)
    rms = (num / den) ** 0.5
    bound = TOL_RMS[dtype] if rms_bound is None else rms_bound
    print(f"{what}: worst {worst:.3g} at {worst_at}, rms {rms:.3g} (bound {bound:.3g})")
    assert rms <= bound, f"{what}: rms error {rms:.3g}, bound {bound:.3g}"
    for rid, rows in ref.items():
        assert all((rid, p) in got for p in rows), f"{what}: {rid} incomplete"


def _trace(regime, reqs):
    make = {"whole": H.trace_whole, "tail": H.trace_decode_tail, "portions": H.trace_portions,
            "mixed": H.trace_mixed}[regime]
    return H.thin_wants(make(reqs), _keep(reqs))


# what a step of the full model launches, by regime (bfloat16)
EXPECTED_KERNELS = {
    "whole": {"prefill_attention_umma2", "qk_norm_rope_kv_write", "add_rmsnorm", "silu_mul"},
    "tail": {"gemm_bf16_cluster", "gemm_bf16_cluster_add_norm", "gemm_bf16_swiglu",
             "gemm_bf16_tcgen05", "decode_attention_persistent"},
}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("regime,page_size", [("whole", 64), ("tail", 64), ("portions", 64),
                                              ("mixed", 64), ("tail", 16), ("mixed", 16)])
def test_replay_at_qwen3_8b_layer_sizes(shape, dtype, regime, page_size):
    """Whole; the last 32 tokens one by one through captured graphs; portions down to two
    tokens; mixed with up to four live requests and the pool at its peak need, so that
    pages are used again.  64-token pages (the engine's default) and 16-token pages."""
    from binfer_b200.csrc import ops
    reqs = _requests(extra=regime == "mixed")
    ref = shape.plain(reqs)
    steps = _trace(regime, reqs)
    runner = shape.runner(dtype, page_size, H.peak_pages(steps, page_size),
                          graphs=regime in ("tail", "mixed"))
    seen = _Names()
    ops.set_profiler(seen)
    try:
        got = H.run_trace(runner, steps)
    finally:
        ops.set_profiler(None)
    assert not runner.cache.requests and all(g.pool.num_held == 0 for g in runner.cache.groups)
    if regime in ("tail", "mixed"):
        assert getattr(runner, "graph_replays", 0) > 0, "no decode step ran from a graph"
    _compare(got, ref, dtype, f"8B sizes/{regime}/page {page_size}",
             shape.reference_rounding_rms(reqs) if dtype == torch.bfloat16 else None)
    if dtype == torch.bfloat16 and regime in EXPECTED_KERNELS:
        missing = EXPECTED_KERNELS[regime] - seen.names
        assert not missing, f"{regime}: kernels that did not run: {sorted(missing)}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_six_requests_decode_together_from_the_bucket_of_eight(shape, dtype):
    """Six requests, prefilled one after the other, then sixteen steps in which all of them
    decode side by side: the graph of bucket 8, two rows of it padding."""
    lens = [150, 40, 97, 64, 33, 120]
    reqs = {f"d{i}": H.random_tokens(n, VOCAB, 31 * i + n) for i, n in enumerate(lens)}
    tail = 16
    keep = lambda rid, p: p >= len(reqs[rid]) - tail - 1   # noqa: E731
    ref = {}
    for rid, toks in reqs.items():
        rows = [p for p in range(len(toks)) if keep(rid, p)]
        lg = P.forward(shape.raw, shape.w64, toks, dtype=torch.float64, rows=rows)
        ref[rid] = {p: lg[i] for i, p in enumerate(rows)}
    steps = []
    for rid, toks in reqs.items():
        n = len(toks) - tail
        steps.append({"step": len(steps), "entries": [
            {"id": rid, "tokens": toks[:n], "want": list(range(n))}], "end": []})
    for i in range(tail):
        steps.append({"step": len(steps), "entries": [
            {"id": rid, "tokens": [toks[len(toks) - tail + i]], "want": [0]}
            for rid, toks in reqs.items()], "end": list(reqs) if i == tail - 1 else []})
    steps = H.thin_wants(steps, keep)
    runner = shape.runner(dtype, 64, H.peak_pages(steps, 64), graphs=True)
    got = H.run_trace(runner, steps)
    assert runner.graph_replays == tail - 1 and list(runner._graphs) == [8]
    bound = None
    if dtype == torch.bfloat16:       # the reference's rounding on the same tokens, as above
        num = den = 0.0
        for rid, toks in reqs.items():
            rows = sorted(ref[rid])
            lg = P.forward(shape.raw, shape.w64, toks, dtype=torch.float64, rows=rows,
                           round_to=torch.bfloat16)
            ex = torch.stack([ref[rid][p] for p in rows])
            num, den = num + float((lg - ex).pow(2).sum()), den + float(ex.pow(2).sum())
        bound = (num / den) ** 0.5
    _compare(got, ref, dtype, "8B sizes/six decoding together", bound)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_a_long_portion_beside_many_decoding_requests(shape, dtype):
    """What a serving step looks like: twenty requests that decode one token each beside a
    600-token portion of another request's prompt (which starts at position 100), in one
    batch: the decode attention over a subset of rows, the prefill attention over the rest,
    the products at 620 token rows.  Then four more such steps with shorter portions."""
    lens = [33 + 3 * i for i in range(20)]
    reqs = {f"s{i}": H.random_tokens(n + 5, VOCAB, 500 + i) for i, n in enumerate(lens)}
    reqs["big"] = H.random_tokens(100 + 600 + 4 * 37, VOCAB, 999)
    keep = lambda rid, p: (p >= len(reqs[rid]) - 6) if rid != "big" else p % 41 == 0   # noqa: E731
    ref = {}
    for rid, toks in reqs.items():
        rows = [p for p in range(len(toks)) if keep(rid, p)]
        lg = P.forward(shape.raw, shape.w64, toks, dtype=torch.float64, rows=rows)
        ref[rid] = {p: lg[i] for i, p in enumerate(rows)}
    steps = []
    for rid, toks in reqs.items():              # the prompts first, each alone
        n = 100 if rid == "big" else len(toks) - 5
        steps.append({"step": len(steps), "entries": [
            {"id": rid, "tokens": toks[:n], "want": list(range(n))}], "end": []})
    at = 100
    for k, portion in enumerate([600, 37, 37, 37, 37]):
        entries = [{"id": "big", "tokens": reqs["big"][at:at + portion],
                    "want": list(range(portion))}]
        at += portion
        for rid, toks in reqs.items():
            if rid != "big":
                entries.append({"id": rid, "tokens": [toks[len(toks) - 5 + k]], "want": [0]})
        steps.append({"step": len(steps), "entries": entries,
                      "end": list(reqs) if k == 4 else []})
    steps = H.thin_wants(steps, keep)
    runner = shape.runner(dtype, 16, H.peak_pages(steps, 16), max_requests=24)
    got = H.run_trace(runner, steps)
    bound = None
    if dtype == torch.bfloat16:
        num = den = 0.0
        for rid, toks in reqs.items():
            rows = sorted(ref[rid])
            lg = P.forward(shape.raw, shape.w64, toks, dtype=torch.float64, rows=rows,
                           round_to=torch.bfloat16)
            ex = torch.stack([ref[rid][p] for p in rows])
            num, den = num + float((lg - ex).pow(2).sum()), den + float(ex.pow(2).sum())
        bound = (num / den) ** 0.5
    _compare(got, ref, dtype, "8B sizes/a long portion beside twenty decoding requests", bound)
