"""Generation through the Python entry point against the plain implementation."""
import pytest
import torch

import helpers as H
import qwen3_plain as P

pytestmark = pytest.mark.gpu


def _engine(d, dtype="float32", **kw):
    from binfer_b200 import Engine
    kw.setdefault("num_pages", 64)
    kw.setdefault("max_seq_len", 256)
    kw.setdefault("max_batch_size", 8)
    return Engine(d, dtype, **kw)


@pytest.mark.parametrize("graphs", [True, False], ids=["graphs", "eager"])
def test_greedy_matches_plain_config_a(cuda_device, tmp_path, graphs):
    """Three prompts of 5/17/33 tokens, 16 greedy tokens each."""
    d = H.make_model_dir(tmp_path, "A")
    raw, w = H.read_model_dir(d)
    prompts = [H.random_tokens(n, raw["vocab_size"], n) for n in (5, 17, 33)]
    want = [P.greedy_generate(raw, w, p, 16) for p in prompts]
    eng = _engine(d, page_size=16, cuda_graphs=graphs)
    got = eng.generate(prompts, max_tokens=16, ignore_eos=True)
    assert got == want
    if graphs:
        assert getattr(eng.runner, "graph_replays", 0) > 0, "decode never ran from a graph"
    assert eng.stats()["pages_free"] == eng.stats()["pages_total"]


def test_single_prompt_and_callback(cuda_device, tmp_path):
    d = H.make_model_dir(tmp_path, "A")
    raw, w = H.read_model_dir(d)
    prompt = H.random_tokens(12, raw["vocab_size"], 5)
    want = P.greedy_generate(raw, w, prompt, 10)
    eng = _engine(d)
    assert eng.generate(prompt, max_tokens=10, ignore_eos=True) == want
    seen = []
    out = eng.generate(prompt, max_tokens=10, ignore_eos=True,
                       on_token=lambda i, t: (seen.append(t), len(seen) < 4)[1])
    assert out == want[:4] and seen == want[:4]


def test_stop_token_is_kept(cuda_device, tmp_path):
    d = H.make_model_dir(tmp_path, "A")
    raw, w = H.read_model_dir(d)
    prompt = H.random_tokens(9, raw["vocab_size"], 2)
    full = P.greedy_generate(raw, w, prompt, 12)
    stop = full[5]
    first = full.index(stop)
    eng = _engine(d)
    assert eng.generate(prompt, max_tokens=12, eos_ids=[stop]) == full[:first + 1]


def test_temperature_config_b_portions_mixed(cuda_device, tmp_path):
    """Four prompts of 1/9/40/70 tokens, prompts cut into portions of 7 beside decoding,
    temperature 0.8 with a fixed seed: every drawn token is what the plain sampler draws
    from the plain logits with the same uniform number, and a request draws the same
    tokens alone as in company."""
    from binfer_b200.sampling import uniform
    d = H.make_model_dir(tmp_path, "B")
    raw, w = H.read_model_dir(d)
    prompts = [H.random_tokens(n, raw["vocab_size"], 40 + n) for n in (1, 9, 40, 70)]
    eng = _engine(d, page_size=8, max_tokens_per_step=7)
    together = eng.generate(prompts, max_tokens=12, temperature=0.8, seed=1234, ignore_eos=True)
    for i, (p, out) in enumerate(zip(prompts, together)):
        logits = P.forward(raw, w, p + out, dtype=torch.float64)
        for n, tok in enumerate(out):
            u = uniform(1234 + i, n)
            assert P.sample(logits[len(p) + n - 1], temperature=0.8, uniform=u) == tok, (i, n)
    alone = _engine(d, page_size=8)
    for i, p in enumerate(prompts):
        assert alone.generate(p, max_tokens=12, temperature=0.8, seed=1234 + i,
                              ignore_eos=True) == together[i]


def test_preemption_recomputes_the_same_tokens(cuda_device, tmp_path):
    """With too few pages for all requests to finish side by side, some are preempted
    and recomputed; the tokens are those of a run with room to spare."""
    d = H.make_model_dir(tmp_path, "B")
    raw, w = H.read_model_dir(d)
    prompts = [H.random_tokens(n, raw["vocab_size"], 7 * n) for n in (20, 22, 18, 25)]
    roomy = _engine(d, page_size=8, num_pages=64)
    want = roomy.generate(prompts, max_tokens=30, temperature=0.7, seed=5, ignore_eos=True)
    assert roomy.stats()["preemptions"] == 0
    tight = _engine(d, page_size=8, num_pages=16)      # 128 tokens for 4 x ~50
    got = tight.generate(prompts, max_tokens=30, temperature=0.7, seed=5, ignore_eos=True)
    assert tight.stats()["preemptions"] > 0
    assert got == want
    assert tight.stats()["pages_free"] == tight.stats()["pages_total"]


def test_bfloat16_generation_matches_plain_within_rounding(cuda_device, tmp_path):
    """bfloat16, graphs and eager: the same tokens both ways, and tokens that the plain
    implementation (float64, on the same stored weights) also ranks first, up to what
    bfloat16 rounding can tell apart."""
    d = H.make_model_dir(tmp_path, "A", torch.bfloat16)
    raw, w = H.read_model_dir(d)
    prompts = [H.random_tokens(n, 256, n) for n in (5, 17, 33)]
    a = _engine(d, "bfloat16").generate(prompts, max_tokens=16, ignore_eos=True)
    b = _engine(d, "bfloat16", cuda_graphs=False).generate(prompts, max_tokens=16, ignore_eos=True)
    assert all(len(x) == 16 for x in a)
    assert a == b
    H.assert_greedy_within_rounding(raw, w, prompts, a)


def test_warm_up_captures_the_decode_graphs_before_the_first_request(cuda_device, tmp_path):
    d = H.make_model_dir(tmp_path, "A")
    raw, w = H.read_model_dir(d)
    prompts = [H.random_tokens(n, raw["vocab_size"], n) for n in (5, 17, 33)]
    want = [P.greedy_generate(raw, w, p, 8) for p in prompts]
    eng = _engine(d, page_size=16)
    eng.warm_up()
    r = eng.runner
    assert sorted(r._graphs) == r._buckets == [1, 2, 4, 8]
    assert all(st["graph"] is not None for st in r._graphs.values())
    assert eng.stats()["pages_free"] == eng.stats()["pages_total"] and not r.cache.requests
    captured = r.graph_captures
    assert eng.generate(prompts, max_tokens=8, ignore_eos=True) == want
    assert r.graph_captures == captured, "a graph was captured while a request waited"
    assert r.graph_replays > 0


def test_cli_generates(cuda_device, tmp_path, capsys):
    from binfer_b200.cli import main
    d = H.make_model_dir(tmp_path, "A")
    raw, w = H.read_model_dir(d)
    prompt = H.random_tokens(7, raw["vocab_size"], 1)
    want = P.greedy_generate(raw, w, prompt, 6)
    rc = main([d, "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "6", "--dtype",
               "fp32", "--ignore-eos", "-q", "--kv-pages", "32"])
    assert rc == 0
    assert capsys.readouterr().out.split() == [str(t) for t in want]


@pytest.mark.parametrize("temperature", [0.0, 0.9])
def test_look_ahead_gives_the_same_tokens(cuda_device, tmp_path, temperature):
    """Launching a step before the last one's ids are read changes nothing: same tokens
    as the synchronous loop, stop tokens honoured, nothing sampled after them kept."""
    d = H.make_model_dir(tmp_path, "B")
    raw, w = H.read_model_dir(d)
    prompts = [H.random_tokens(n, raw["vocab_size"], 3 * n) for n in (4, 31, 9, 17)]
    kw = dict(max_tokens=24, temperature=temperature, seed=11, ignore_eos=True)
    sync = _engine(d, page_size=8, look_ahead=False)
    want = sync.generate(prompts, **kw)
    ahead = _engine(d, page_size=8, look_ahead=True)
    assert ahead.generate(prompts, **kw) == want
    # a stop token in the middle of a request's output
    stop = want[1][7]
    cut = [o[:o.index(stop) + 1] if stop in o else o for o in want]
    kw2 = dict(kw, ignore_eos=False, eos_ids=[stop])
    assert _engine(d, page_size=8, look_ahead=False).generate(prompts, **kw2) == cut
    eng = _engine(d, page_size=8, look_ahead=True)
    assert eng.generate(prompts, **kw2) == cut
    assert eng.stats()["pages_free"] == eng.stats()["pages_total"] and not eng.has_work()
    # few pages: preemption switches the look-ahead off where it must, tokens stay the same
    tight = _engine(d, page_size=8, num_pages=14, look_ahead=True)
    assert tight.generate(prompts, **kw) == want
    assert tight.stats()["preemptions"] > 0


def test_continuous_batching_at_qwen3_1p7b_layer_sizes(cuda_device, tmp_path):
    """The scheduler at real layer sizes (two layers of the Qwen3-1.7B shape): eight requests
    with prompts of 128 to 512 tokens and 160 output tokens each, submitted at once, a step
    budget of 512 tokens (so prompts come in portions beside decoding requests), and a pool
    that holds all the prompts but not what they grow into, so that requests are preempted
    and recomputed.  float32: the
    tokens are those of a run with room to spare (every sum's order depends on the position
    only).  bfloat16, same pool: tokens that the plain implementation also ranks first, up
    to what bfloat16 rounding can tell apart."""
    from binfer_b200 import Engine, Qwen3Config
    from binfer_b200.weights import write_model_dir
    cfg = Qwen3Config.from_dict(H.QWEN3_1P7B_TWO_LAYERS)
    d = write_model_dir(cfg, str(tmp_path / "qwen3_1p7b_two_layers"), seed=17, std=0.02,
                        norm_std=0.05, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(3)
    lens = torch.randint(128, 513, (8,), generator=g).tolist()
    prompts = [H.random_tokens(n, cfg.vocab_size, 1000 + n) for n in lens]
    kw = dict(page_size=64, max_seq_len=1024, max_batch_size=8, max_tokens_per_step=512)
    n_out = 160
    need = sum(-(-(n + n_out) // 64) for n in lens)
    few = sum(-(-n // 64) for n in lens) + 10        # the prompts, a page each to grow into
    roomy = Engine(d, "float32", num_pages=need + 8, **kw)
    want = roomy.generate(prompts, max_tokens=n_out, ignore_eos=True)
    assert roomy.stats()["preemptions"] == 0
    del roomy
    tight = Engine(d, "float32", num_pages=few, **kw)
    got = tight.generate(prompts, max_tokens=n_out, ignore_eos=True)
    assert tight.stats()["preemptions"] > 0
    assert got == want
    assert tight.stats()["pages_free"] == tight.stats()["pages_total"]
    del tight
    torch.cuda.empty_cache()
    eng = Engine(d, "bfloat16", num_pages=few, **kw)
    out = eng.generate(prompts, max_tokens=n_out, ignore_eos=True)
    assert eng.stats()["preemptions"] > 0 and all(len(o) == n_out for o in out)
    assert eng.runner.graph_replays > 0
    raw, w = H.read_model_dir(d)
    w = {k: t.to(torch.float64) for k, t in w.items()}
    H.assert_greedy_within_rounding(raw, w, prompts[:3], out[:3])
