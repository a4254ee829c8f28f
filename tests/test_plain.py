"""The plain implementation checked against itself and against a second, independent
restatement of the same formulas (no GPU)."""
import json
import math
import os

import pytest
import torch

import helpers as H
import qwen3_plain as P


def test_rms_norm_formula():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    y = P.rms_norm(x, w, 0.0)
    assert torch.allclose(y, torch.tensor([[3 / math.sqrt(12.5) * 2, 4 / math.sqrt(12.5) * 0.5]],
                                          dtype=torch.float64))


def test_rope_is_a_rotation_that_depends_on_relative_position():
    d = 8
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, 1, d, generator=g, dtype=torch.float64)
    k = torch.randn(1, 1, d, generator=g, dtype=torch.float64)

    def dot(pq, pk):
        a = P.apply_rope(q, P.rope_angles(torch.tensor([pq]), d, 100.0))
        b = P.apply_rope(k, P.rope_angles(torch.tensor([pk]), d, 100.0))
        return float((a * b).sum())

    assert abs(dot(5, 3) - dot(12, 10)) < 1e-5
    assert abs(float(P.apply_rope(q, P.rope_angles(torch.tensor([9]), d, 100.0)).norm())
               - float(q.norm())) < 1e-12
    # position 0 leaves the vector alone; pairs are (i, i + d/2)
    assert torch.equal(P.apply_rope(q, P.rope_angles(torch.tensor([0]), d, 100.0)), q)
    e = torch.zeros(1, 1, d, dtype=torch.float64)
    e[0, 0, 0] = 1
    r = P.apply_rope(e, P.rope_angles(torch.tensor([1]), d, 100.0))
    assert abs(float(r[0, 0, 0]) - math.cos(1.0)) < 1e-7 and abs(float(r[0, 0, 4]) - math.sin(1.0)) < 1e-7


def test_attention_against_explicit_loops():
    g = torch.Generator().manual_seed(1)
    T, nh, nkv, d, window = 9, 4, 2, 6, 4
    q = torch.randn(T, nh, d, generator=g, dtype=torch.float64)
    k = torch.randn(T, nkv, d, generator=g, dtype=torch.float64)
    v = torch.randn(T, nkv, d, generator=g, dtype=torch.float64)
    for w in (None, window):
        out = P.causal_attention(q, k, v, 0.3, w)
        for t in range(T):
            for h in range(nh):
                kv = h // (nh // nkv)
                js = [j for j in range(t + 1) if w is None or j > t - w]
                s = torch.tensor([float(q[t, h] @ k[j, kv]) * 0.3 for j in js], dtype=torch.float64)
                p = torch.exp(s - s.max())
                p = p / p.sum()
                want = sum(p[i] * v[j, kv] for i, j in enumerate(js))
                assert torch.allclose(out[t, h], want, atol=1e-12)


@pytest.mark.parametrize("which", ["A", "B", "W"])
def test_forward_is_causal_and_deterministic(tmp_path, which):
    d = H.make_model_dir(tmp_path, which)
    raw, w = H.read_model_dir(d)
    ids = H.random_tokens(40, raw["vocab_size"], 1)
    full = P.forward(raw, w, ids, torch.float64)
    assert full.shape == (40, raw["vocab_size"])
    part = P.forward(raw, w, ids[:17], torch.float64)
    assert torch.allclose(full[:17], part, atol=1e-12)
    changed = list(ids)
    changed[30] = (changed[30] + 1) % raw["vocab_size"]
    assert torch.allclose(P.forward(raw, w, changed, torch.float64)[:30], full[:30], atol=1e-12)
    assert not torch.allclose(P.forward(raw, w, changed, torch.float64)[30:], full[30:], atol=1e-6)
    assert H.rel_err(P.forward(raw, w, ids, torch.float32), full) < 2e-5


def test_window_changes_the_result_only_past_the_window(tmp_path):
    d = H.make_model_dir(tmp_path, "W")
    raw, w = H.read_model_dir(d)
    ids = H.random_tokens(60, raw["vocab_size"], 2)
    with_w = P.forward(raw, w, ids, torch.float64)
    no_w = P.forward({**raw, "layer_types": ["full_attention"] * 4}, w, ids, torch.float64)
    assert torch.allclose(with_w[:24], no_w[:24], atol=1e-12)       # window 24 not yet passed
    assert not torch.allclose(with_w[40:], no_w[40:], atol=1e-6)


def test_tied_head_uses_the_embedding_table(tmp_path):
    d = H.make_model_dir(tmp_path, "A")
    raw, w = H.read_model_dir(d)
    ids = [1, 2, 3]
    a = P.forward(raw, w, ids, torch.float64)
    w2 = dict(w)
    w2["lm_head.weight"] = w["model.embed_tokens.weight"] * 2
    assert torch.allclose(P.forward({**raw, "tie_word_embeddings": False}, w2, ids, torch.float64),
                          2 * a, atol=1e-12)


def test_golden_logits_of_the_plain_implementation(tmp_path):
    """Guards the oracle itself against an accidental change (made by tests/golden/make_golden.py)."""
    path = os.path.join(os.path.dirname(__file__), "golden", "plain_tiny.json")
    with open(path) as f:
        gold = json.load(f)
    for which, g in gold.items():
        d = H.make_model_dir(tmp_path, which)
        raw, w = H.read_model_dir(d)
        lg = P.forward(raw, w, g["tokens"], torch.float64)
        got = lg[-1, :8].tolist()
        assert max(abs(a - b) for a, b in zip(got, g["last_logits_first8"])) < 1e-9
        assert int(lg[-1].argmax()) == g["argmax"]


# ---------------------------------------------------------------------- the sampler
def test_sampler_greedy_is_first_argmax():
    lg = torch.tensor([0.1, 2.0, 2.0, -1.0])
    assert P.sample(lg, 0.0) == 1


def test_sampler_top_k_top_p_and_penalty():
    lg = torch.tensor([3.0, 2.0, 1.0, 0.0, -1.0])
    assert {P.sample(lg, 1.0, top_k=2, uniform=u / 10) for u in range(10)} <= {0, 1}
    assert {P.sample(lg, 1.0, top_p=0.5, uniform=u / 10) for u in range(10)} == {0}
    p = torch.softmax(lg.double(), 0)
    assert P.sample(lg, 1.0, uniform=float(p[0]) - 1e-9) == 0
    assert P.sample(lg, 1.0, uniform=float(p[0]) + 1e-9) == 1
    assert P.sample(lg, 1.0, uniform=0.999999999) == 4
    assert P.sample(torch.tensor([1.0, 3.0, 2.9]), 0.0, repetition_penalty=1.5, generated=[1]) == 2
