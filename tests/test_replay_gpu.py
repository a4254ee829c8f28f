"""Replay on the GPU against the plain implementation: whole, decoded tail, portions, mixed.

Every regime must give, at every position, the logits that the plain whole-sequence
implementation gives; float32 within float32 rounding, bfloat16 within bfloat16
rounding of the activations (the plain side reads the same bfloat16 weights).
"""
import pytest
import torch

import helpers as H
import qwen3_plain as P

pytestmark = pytest.mark.gpu

# largest |difference| / largest |reference logit|
TOL = {torch.float32: 2e-5, torch.bfloat16: 3e-2}
# and root-mean-square of the difference over that of the reference
TOL_RMS = {torch.float32: 5e-6, torch.bfloat16: 1e-2}

LENGTHS = {"A": [5, 17, 33, 70], "B": [1, 9, 40, 70], "W": [3, 30, 64, 101],
           "M": [2, 45, 150, 333], "F": [3, 40, 70, 130], "V": [4, 160, 333, 500],
           "O": [2, 37, 90, 140]}


def _requests(which, extra=()):
    vocab = H.TINY[which]["raw"]["vocab_size"]
    lens = list(LENGTHS[which]) + list(extra)
    return {f"r{i}": H.random_tokens(n, vocab, 100 * i + n) for i, n in enumerate(lens)}


@pytest.fixture(scope="module")
def plain_logits(tmp_path_factory):
    """Reference logits per (config, dtype, request), computed once in float64."""
    cache = {}

    def get(which, dtype, reqs):
        key = (which, dtype)
        d = H.make_model_dir(tmp_path_factory.getbasetemp(), which, dtype)
        raw, w = H.read_model_dir(d)
        out = cache.setdefault(key, {})
        for rid, toks in reqs.items():
            k = (rid, tuple(toks))
            if k not in out:
                out[k] = P.forward(raw, w, toks, dtype=torch.float64)
        return d, {rid: out[(rid, tuple(toks))] for rid, toks in reqs.items()}

    return get


def _runner(model_dir, dtype, page_size, num_pages):
    from binfer_b200.engine import make_env, make_runner, model_from_dir
    env = make_env(dtype)
    model = model_from_dir(model_dir, env)
    return make_runner(model, env, page_size=page_size, num_pages=num_pages, max_requests=8)


def _compare(got, ref, dtype, what):
    assert got, "the trace produced no logits"
    worst, worst_at = 0.0, None
    for (rid, pos), row in got.items():
        e = H.rel_err(row, ref[rid][pos])
        if e > worst:
            worst, worst_at = e, (rid, pos)
    assert worst <= TOL[dtype], f"{what}: worst relative error {worst:.3g} at {worst_at}"
    g = torch.stack([row for row in got.values()])
    r = torch.stack([ref[rid][pos] for (rid, pos) in got])
    assert H.rel_rms(g, r) <= TOL_RMS[dtype], f"{what}: rms error {H.rel_rms(g, r):.3g}"
    # every position of every request was produced
    for rid, lg in ref.items():
        assert all((rid, p) in got for p in range(lg.shape[0])), f"{what}: {rid} incomplete"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("which", ["A", "B", "W", "M", "V"])
@pytest.mark.parametrize("regime", ["whole", "tail", "portions", "mixed"])
def test_replay(cuda_device, plain_logits, which, dtype, regime):
    extra = (55, 61) if regime == "mixed" else ()
    reqs = _requests(which, extra)
    model_dir, ref = plain_logits(which, dtype, reqs)
    steps = {"whole": H.trace_whole, "tail": H.trace_decode_tail,
             "portions": H.trace_portions, "mixed": H.trace_mixed}[regime](reqs)
    ps = H.TINY[which]["page_size"]
    # exactly the peak need: every page that is given back is handed out again
    runner = _runner(model_dir, dtype, ps, H.peak_pages(steps, ps))
    got = H.run_trace(runner, steps)
    assert not runner.cache.requests, "a finished request still holds pages"
    assert all(g.pool.num_held == 0 for g in runner.cache.groups)
    _compare(got, ref, dtype, f"{which}/{regime}")


@pytest.mark.parametrize("which", ["A", "B", "W", "M", "V"])
def test_regimes_agree_bitwise_in_float32(cuda_device, plain_logits, which):
    """In float32 the order of every sum is fixed by the position alone, so cutting
    and batching change nothing at all."""
    reqs = _requests(which)
    model_dir, _ = plain_logits(which, torch.float32, reqs)
    ps = H.TINY[which]["page_size"]
    outs = []
    for make in (H.trace_whole, H.trace_decode_tail, H.trace_portions, H.trace_mixed):
        steps = make(reqs)
        outs.append(H.run_trace(_runner(model_dir, torch.float32, ps, H.peak_pages(steps, ps)),
                                steps))
    for other in outs[1:]:
        for key, row in outs[0].items():
            assert torch.equal(row, other[key]), f"{which}: logits at {key} depend on the cut"


def test_long_decoding(cuda_device, plain_logits):
    """A short prompt, then 300 tokens one by one (across many pages)."""
    which, dtype = "B", torch.float32
    vocab = H.TINY[which]["raw"]["vocab_size"]
    reqs = {"long": H.random_tokens(304, vocab, 7)}
    model_dir, ref = plain_logits(which, dtype, reqs)
    steps = H.trace_decode_tail(reqs, tail=300)
    runner = _runner(model_dir, dtype, 8, H.peak_pages(steps, 8))
    _compare(H.run_trace(runner, steps), ref, dtype, "long decoding")


def test_first_tokens(cuda_device, plain_logits):
    """The first tokens of a sequence, one per step from the very start."""
    for which in ("A", "B"):
        vocab = H.TINY[which]["raw"]["vocab_size"]
        reqs = {"s": H.random_tokens(6, vocab, 3)}
        model_dir, ref = plain_logits(which, torch.float32, reqs)
        steps = H.trace_decode_tail(reqs, tail=5)
        runner = _runner(model_dir, torch.float32, H.TINY[which]["page_size"], 4)
        _compare(H.run_trace(runner, steps), ref, torch.float32, f"{which}/first tokens")


@pytest.mark.parametrize("which,dtype", [("M", torch.float32), ("M", torch.bfloat16),
                                         ("F", torch.bfloat16)], ids=["M-f32", "M-bf16", "F-bf16"])
def test_replay_through_captured_decode_steps(cuda_device, plain_logits, which, dtype):
    """Steps of single tokens replayed from CUDA graphs (padded to a bucket, block tables of
    full width) give what eager steps give.  (F: with the products that prepare the next
    norm, the cluster kernels and their dependent launches inside the graph.)"""
    reqs = _requests(which, (55, 61))
    model_dir, ref = plain_logits(which, dtype, reqs)
    ps = H.TINY[which]["page_size"]
    for make in (H.trace_decode_tail, H.trace_mixed):
        steps = make(reqs)
        runner = _runner(model_dir, dtype, ps, H.peak_pages(steps, ps))
        runner.enable_decode_graphs(max_batch=8, max_seq_len=512)
        got = H.run_trace(runner, steps)
        assert getattr(runner, "graph_replays", 0) > 0
        _compare(got, ref, dtype, f"{which}/graphs/{make.__name__}")


class _Names:
    """A profiler stand-in that only records which kernels were launched."""
    def __init__(self):
        self.names = set()

    def begin(self, name):
        self.names.add(name)

    def end(self, name):
        pass


@pytest.mark.parametrize("which", ["F", "O"])
@pytest.mark.parametrize("regime", ["tail", "mixed"])
def test_replay_with_products_that_prepare_the_next_norm(cuda_device, plain_logits, regime, which):
    """A model wide enough for the decode step's cluster products: steps of few tokens run
    the output and down projections with the add into the stream and the next norm in their
    epilogue, and the norm's factor is applied after the next product.  Same logits as the
    plain implementation, and (to bfloat16 rounding) as the same steps without the fusion."""
    from binfer_b200.csrc import ops
    import importlib
    lin = importlib.import_module("binfer_b200.parts.linear")
    dtype = torch.bfloat16
    reqs = _requests(which, (55, 61) if regime == "mixed" else ())
    model_dir, ref = plain_logits(which, dtype, reqs)
    steps = {"tail": H.trace_decode_tail, "mixed": H.trace_mixed}[regime](reqs)
    ps = H.TINY[which]["page_size"]
    outs = []
    for fuse in (True, False):
        lin.FUSE_NORM = fuse
        seen = _Names()
        ops.set_profiler(seen)
        try:
            got = H.run_trace(_runner(model_dir, dtype, ps, H.peak_pages(steps, ps)), steps)
        finally:
            ops.set_profiler(None)
            lin.FUSE_NORM = True
        assert ("gemm_bf16_cluster_add_norm" in seen.names) == fuse
        if fuse:        # the factor is applied by what follows the next product
            assert "silu_mul_scaled" in seen.names or "gemm_bf16_swiglu" in seen.names
        _compare(got, ref, dtype, f"{which}/{regime}/fused={fuse}")
        outs.append(got)
    worst = max(H.rel_err(outs[0][k], outs[1][k]) for k in outs[0])
    assert worst <= TOL[dtype], f"fused and unfused steps differ by {worst:.3g}"


@pytest.mark.parametrize("which", ["F", "O", "V", "M"])
@pytest.mark.parametrize("regime", ["tail", "mixed"])
def test_replay_with_the_projection_that_stores_into_the_pages(cuda_device, plain_logits, regime,
                                                               which):
    """Steps of few tokens run the q/k/v projection with the head norms, the rotation and the
    store into the pages in its epilogue (switched on here, also where its tiles would leave
    most SMs idle).  Same logits as the plain implementation, and (to bfloat16 rounding) as the
    same steps with the separate kernels; V has windows, whose pages are given back."""
    from binfer_b200.csrc import ops
    import importlib
    att = importlib.import_module("binfer_b200.parts.attention")
    dtype = torch.bfloat16
    reqs = _requests(which, (55, 61) if regime == "mixed" else ())
    model_dir, ref = plain_logits(which, dtype, reqs)
    steps = {"tail": H.trace_decode_tail, "mixed": H.trace_mixed}[regime](reqs)
    ps = H.TINY[which]["page_size"]
    outs = []
    before = att.FUSE_QKV, att.FUSE_QKV_FILL
    for fuse in (True, False):
        att.FUSE_QKV, att.FUSE_QKV_FILL = fuse, 0.0
        seen = _Names()
        ops.set_profiler(seen)
        try:
            got = H.run_trace(_runner(model_dir, dtype, ps, H.peak_pages(steps, ps)), steps)
        finally:
            ops.set_profiler(None)
            att.FUSE_QKV, att.FUSE_QKV_FILL = before
        assert ("gemm_bf16_cluster_qkv" in seen.names) == fuse
        _compare(got, ref, dtype, f"{which}/{regime}/fused={fuse}")
        outs.append(got)
    worst = max(H.rel_err(outs[0][k], outs[1][k]) for k in outs[0])
    assert worst <= TOL[dtype], f"fused and separate kernels differ by {worst:.3g}"


@pytest.mark.parametrize("which", ["F", "O", "M"])
def test_replay_with_the_activation_in_the_projection(cuda_device, plain_logits, which):
    """Steps of few tokens run the gate/up projection with the activation in its epilogue.
    Same logits as the plain implementation, and (to bfloat16 rounding) as the same steps
    with the product and the activation as two kernels."""
    from binfer_b200.csrc import ops
    import importlib
    mlp = importlib.import_module("binfer_b200.parts.mlp")
    dtype = torch.bfloat16
    reqs = _requests(which, (55, 61))
    model_dir, ref = plain_logits(which, dtype, reqs)
    steps = H.trace_mixed(reqs)
    ps = H.TINY[which]["page_size"]
    outs = []
    before = mlp.FUSE_SWIGLU, mlp.FUSE_SWIGLU_FILL
    for fuse in (True, False):
        mlp.FUSE_SWIGLU, mlp.FUSE_SWIGLU_FILL = fuse, 0.0     # (also where few SMs get a tile)
        seen = _Names()
        ops.set_profiler(seen)
        try:
            got = H.run_trace(_runner(model_dir, dtype, ps, H.peak_pages(steps, ps)), steps)
        finally:
            ops.set_profiler(None)
            mlp.FUSE_SWIGLU, mlp.FUSE_SWIGLU_FILL = before
        assert ("gemm_bf16_swiglu" in seen.names) == fuse
        _compare(got, ref, dtype, f"{which}/mixed/swiglu={fuse}")
        outs.append(got)
    worst = max(H.rel_err(outs[0][k], outs[1][k]) for k in outs[0])
    assert worst <= TOL[dtype], f"fused and separate kernels differ by {worst:.3g}"


def test_long_context_bfloat16(cuda_device, plain_logits):
    """A prompt of 2600 tokens (portions of 2048 and the rest), then 40 tokens one by one: the
    tcgen05 prefill kernels over many key tiles, the decode kernels over 21 splits, and the
    graph-captured step, against the plain implementation."""
    which, dtype = "M", torch.bfloat16
    vocab = H.TINY[which]["raw"]["vocab_size"]
    reqs = {"long": H.random_tokens(2640, vocab, 17)}
    model_dir, ref = plain_logits(which, dtype, reqs)
    toks = reqs["long"]
    steps = [{"step": 0, "entries": [{"id": "long", "tokens": toks[:2048], "want": [0, 2047]}], "end": []},
             {"step": 1, "entries": [{"id": "long", "tokens": toks[2048:2600],
                                      "want": [0, 551]}], "end": []}]
    for i in range(2600, 2640):
        steps.append({"step": len(steps), "entries": [{"id": "long", "tokens": [toks[i]], "want": [0]}],
                      "end": ["long"] if i == 2639 else []})
    runner = _runner(model_dir, dtype, 64, H.peak_pages(steps, 64))
    runner.enable_decode_graphs(max_batch=2, max_seq_len=4096)
    got = H.run_trace(runner, steps)
    worst = max(H.rel_err(row, ref["long"][pos]) for (rid, pos), row in got.items())
    assert len(got) == 44 and worst <= TOL[dtype], worst


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_logits_alone_and_in_company(cuda_device, plain_logits, dtype):
    """A request decodes ten tokens alone, and again with a 39-token portion of another
    request's prompt in each of its steps.  float32: the same bits (every sum's order depends
    on the position only).  bfloat16: which kernel runs a product depends on how many tokens
    the step holds (the split-K cluster kernels up to 32 tokens, the library beyond; decode
    and prefill attention kernels), so the bits differ; the logits agree within the bound
    that both are held to against the plain implementation."""
    which = "F"
    vocab = H.TINY[which]["raw"]["vocab_size"]
    reqs = {"a": H.random_tokens(70, vocab, 5), "b": H.random_tokens(39 * 10, vocab, 6)}
    model_dir, ref = plain_logits(which, dtype, reqs)
    a, b = reqs["a"], reqs["b"]
    first = {"step": 0, "entries": [{"id": "a", "tokens": a[:60], "want": [59]}], "end": []}
    alone, company = [first], [dict(first)]
    for i in range(10):
        last = i == 9
        alone.append({"step": i + 1, "entries": [{"id": "a", "tokens": [a[60 + i]], "want": [0]}],
                      "end": ["a"] if last else []})
        company.append({"step": i + 1, "entries": [
            {"id": "b", "tokens": b[39 * i:39 * (i + 1)], "want": [38]},
            {"id": "a", "tokens": [a[60 + i]], "want": [0]}], "end": ["a", "b"] if last else []})
    ps = H.TINY[which]["page_size"]
    outs = [H.run_trace(_runner(model_dir, dtype, ps, H.peak_pages(st, ps)), st)
            for st in (alone, company)]
    for key, row in outs[0].items():
        assert H.rel_err(row, ref[key[0]][key[1]]) <= TOL[dtype]
        other = outs[1][key]
        if dtype == torch.float32:
            assert torch.equal(row, other), f"float32 logits at {key} depend on the company"
        else:
            assert H.rel_err(other, row) <= TOL[dtype], f"logits at {key} differ in company"
    for key, row in outs[1].items():
        assert H.rel_err(row, ref[key[0]][key[1]]) <= TOL[dtype]
