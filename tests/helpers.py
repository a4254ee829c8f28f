"""Shared by the tests: tiny configurations, model folders in temporary places, traces."""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from binfer_b200.config import Qwen3Config
from binfer_b200.weights import TensorSource, write_model_dir

# Two tiny configurations that differ in every size and option, and a third with a window.
TINY_A = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=64,
    num_attention_heads=4, num_key_value_heads=2, intermediate_size=128, vocab_size=256,
    rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, use_sliding_window=False,
    max_position_embeddings=512, hidden_act="silu", attention_bias=False)          # head_dim = 64/4
TINY_B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=3, hidden_size=96,
    num_attention_heads=6, num_key_value_heads=1, head_dim=32, intermediate_size=160,
    vocab_size=300, rope_theta=1e6, rms_norm_eps=1e-5, tie_word_embeddings=False,
    use_sliding_window=False, max_position_embeddings=1024, hidden_act="silu",
    attention_bias=False)
TINY_W = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=4, hidden_size=80,
    num_attention_heads=5, num_key_value_heads=5, head_dim=48, intermediate_size=112,
    vocab_size=270, rope_theta=50000.0, rms_norm_eps=3e-6, tie_word_embeddings=False,
    use_sliding_window=True, sliding_window=24,
    layer_types=["full_attention", "sliding_attention", "sliding_attention", "full_attention"],
    max_position_embeddings=2048, hidden_act="silu", attention_bias=False)

# head size 128 and pages of 16: the sizes the TMA / tcgen05 kernels are written for
TINY_M = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=256,
    num_attention_heads=4, num_key_value_heads=2, head_dim=128, intermediate_size=512,
    vocab_size=500, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False,
    use_sliding_window=False, max_position_embeddings=4096, hidden_act="silu",
    attention_bias=False)

# the same sizes with a window on two of three layers: the TMA / tcgen05 attention kernels
# with keys that fall out of the window, and pages that are given back while a request runs
TINY_V = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=3, hidden_size=256,
    num_attention_heads=4, num_key_value_heads=2, head_dim=128, intermediate_size=384,
    vocab_size=410, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=True,
    use_sliding_window=True, sliding_window=150,
    layer_types=["sliding_attention", "full_attention", "sliding_attention"],
    max_position_embeddings=4096, hidden_act="silu", attention_bias=False)

# sizes that are no power of two at the scale where the decode step's cluster products, the
# persistent decode attention and the tcgen05 head product run: a width of 1536, 4480 inner
# features, a vocabulary of 5001.  (One layer: at this width two layers' bfloat16 rounding
# alone, with every product on the library, is 1.05e-2 of the logits' rms, over the bound
# that the other configurations are held to.)
TINY_O = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=1, hidden_size=1536,
    num_attention_heads=16, num_key_value_heads=2, head_dim=128, intermediate_size=4480,
    vocab_size=5001, rope_theta=5e5, rms_norm_eps=2e-6, tie_word_embeddings=False,
    use_sliding_window=False, max_position_embeddings=4096, hidden_act="silu",
    attention_bias=False)

# wide enough (2048 inputs to the output and down projections) for the decode step's
# split-K cluster products, and with them the products that prepare the next norm
TINY_F = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=3, hidden_size=1024,
    num_attention_heads=16, num_key_value_heads=4, head_dim=128, intermediate_size=2048,
    vocab_size=600, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False,
    use_sliding_window=False, max_position_embeddings=4096, hidden_act="silu",
    attention_bias=False)

# the layer sizes of the Qwen3-8B shape (hidden 4096, 32/8 heads of 128, 12288 inner
# features, an untied head over 151936 words) with fewer layers: two.  What a decode or a
# prefill step of the full model launches, kernel for kernel, but small enough to compare
# with the plain implementation.
QWEN3_8B_TWO_LAYERS = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=4096,
    num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
    vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False,
    use_sliding_window=False, max_position_embeddings=40960, hidden_act="silu",
    attention_bias=False)

# the layer sizes of the Qwen3-1.7B shape (tied head), two layers of its 28
QWEN3_1P7B_TWO_LAYERS = dict(
    QWEN3_8B_TWO_LAYERS, hidden_size=2048, num_attention_heads=16, num_key_value_heads=8,
    intermediate_size=6144, tie_word_embeddings=True)

# for the smoke test: small, but of the sizes that a decode step's tcgen05 kernels take
# (2048 inputs to every projection, heads of 128, a head product over more than 65536 words)
SMOKE_WIDE = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=2048,
    num_attention_heads=16, num_key_value_heads=4, head_dim=128, intermediate_size=3072,
    vocab_size=66001, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=True,
    use_sliding_window=False, max_position_embeddings=4096, hidden_act="silu",
    attention_bias=False)

TINY = {
    "S": dict(raw=SMOKE_WIDE, std=0.02, norm_std=0.05, page_size=64, seed=88),
    "O": dict(raw=TINY_O, std=0.03, norm_std=0.05, page_size=64, seed=77),
    "V": dict(raw=TINY_V, std=0.05, norm_std=0.02, page_size=32, seed=66),
    "F": dict(raw=TINY_F, std=0.03, norm_std=0.05, page_size=64, seed=55),
    "M": dict(raw=TINY_M, std=0.05, norm_std=0.02, page_size=16, seed=44),
    "A": dict(raw=TINY_A, std=0.02, norm_std=0.01, page_size=16, seed=11),
    "B": dict(raw=TINY_B, std=0.05, norm_std=0.05, page_size=8, seed=22),
    "W": dict(raw=TINY_W, std=0.04, norm_std=0.03, page_size=4, seed=33),
}


def make_model_dir(tmp_path, which: str, dtype=torch.float32) -> str:
    t = TINY[which]
    cfg = Qwen3Config.from_dict(t["raw"])
    d = os.path.join(str(tmp_path), f"tiny_{which}_{str(dtype).split('.')[-1]}")
    write_model_dir(cfg, d, seed=t["seed"], std=t["std"], norm_std=t["norm_std"], dtype=dtype)
    return d


def read_model_dir(d: str) -> Tuple[dict, Dict[str, torch.Tensor]]:
    with open(os.path.join(d, "config.json")) as f:
        raw = json.load(f)
    src = TensorSource.from_dir(d)
    w = {n: src.get(n).clone() for n in src.shapes}
    src.close()
    return raw, w


def random_tokens(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def rel_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    """Largest absolute difference over the largest reference magnitude."""
    return float((got.double() - ref.double()).abs().max() / ref.double().abs().max())


def rel_rms(got: torch.Tensor, ref: torch.Tensor) -> float:
    d = (got.double() - ref.double())
    return float(d.pow(2).mean().sqrt() / ref.double().pow(2).mean().sqrt())


def assert_greedy_within_rounding(raw, w, prompts, outs, bound=3e-2):
    """Every generated token is the plain implementation's choice at its place, given the
    tokens before it, or, where the plain logits of the best tokens lie closer together than
    bfloat16 rounding can tell apart (``bound`` of the largest logit), one of those."""
    import qwen3_plain as P
    for p, out in zip(prompts, outs):
        logits = P.forward(raw, w, list(p) + list(out), dtype=torch.float64)
        for n, tok in enumerate(out):
            row = logits[len(p) - 1 + n]
            slack = bound * float(row.abs().max())
            assert float(row[tok]) >= float(row.max()) - slack, (
                f"token {n} of a prompt of {len(p)}: {tok} has plain logit {float(row[tok]):.4f}, "
                f"the best ({int(row.argmax())}) {float(row.max()):.4f}")


# ------------------------------------------------------------------------ traces
def trace_whole(reqs: Dict[str, List[int]]) -> List[dict]:
    """Each request alone and whole, logits wanted everywhere."""
    steps = []
    for i, (rid, toks) in enumerate(reqs.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks,
                                              "want": list(range(len(toks)))}], "end": [rid]})
    return steps


def trace_decode_tail(reqs: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps, s = [], 0
    for rid, toks in reqs.items():
        n = max(1, len(toks) - tail)
        steps.append({"step": s, "entries": [{"id": rid, "tokens": toks[:n],
                                              "want": list(range(n))}], "end": []})
        s += 1
        for i in range(n, len(toks)):
            steps.append({"step": s, "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}],
                          "end": [rid] if i == len(toks) - 1 else []})
            s += 1
        if n == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def trace_portions(reqs: Dict[str, List[int]], sizes: Sequence[int] = (7, 5, 3, 2, 11, 2, 16, 9)
                   ) -> List[dict]:
    """Portions of changing size, down to two tokens."""
    steps, s, k = [], 0, 0
    for rid, toks in reqs.items():
        a = 0
        while a < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - a)
            k += 1
            steps.append({"step": s, "entries": [{"id": rid, "tokens": toks[a:a + n],
                                                  "want": list(range(n))}],
                          "end": [rid] if a + n == len(toks) else []})
            a += n
            s += 1
    return steps


def trace_mixed(reqs: Dict[str, List[int]], max_live: int = 4, tail: int = 10,
                sizes: Sequence[int] = (7, 2, 13, 5, 3, 9), skip_every: int = 5) -> List[dict]:
    """Up to ``max_live`` requests at a time: portions of some beside decoded tokens of
    others; a request sits out a step now and then; finished ones make room for new ones."""
    waiting = list(reqs.items())
    live: List[List] = []          # [rid, tokens, done]
    steps, s, k = [], 0, 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live.append([rid, toks, 0])
            if len(live) < max_live and s % 2 == 0:
                break               # stagger arrivals
        entries, end = [], []
        for j, r in enumerate(live):
            rid, toks, done = r
            if (s + j) % skip_every == skip_every - 1 and len(live) > 1:
                continue            # this request sits the step out
            left = len(toks) - done
            n = 1 if left <= tail else min(sizes[k % len(sizes)], left - tail)
            k += 1
            entries.append({"id": rid, "tokens": toks[done:done + n], "want": list(range(n))})
            r[2] = done + n
            if r[2] == len(toks):
                end.append(rid)
        if entries:
            steps.append({"step": s, "entries": entries, "end": end})
        live = [r for r in live if r[2] < len(r[1])]
        s += 1
    return steps


def thin_wants(steps: List[dict], keep) -> List[dict]:
    """The same steps with logits wanted only where ``keep(request, position)`` says so."""
    pos: Dict[str, int] = {}
    out = []
    for st in steps:
        entries = []
        for e in st["entries"]:
            a = pos.get(e["id"], 0)
            entries.append(dict(e, want=[w for w in e["want"] if keep(e["id"], a + w)]))
            pos[e["id"]] = a + len(e["tokens"])
        for rid in st["end"]:
            pos.pop(rid, None)
        out.append(dict(st, entries=entries))
    return out


def peak_pages(steps: List[dict], page_size: int) -> int:
    """Most pages held at once by a full-attention cache group while replaying ``steps``."""
    held: Dict[str, int] = {}
    peak = 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // page_size) for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return peak


def run_trace(runner, steps: List[dict]) -> Dict[Tuple[str, int], torch.Tensor]:
    """Replay ``steps`` on a ModelRunner; logits by (request, position), on the CPU."""
    from binfer_b200.engine.runner import StepItem
    pos: Dict[str, int] = {}
    out: Dict[Tuple[str, int], torch.Tensor] = {}
    for st in steps:
        items = []
        for e in st["entries"]:
            if e["id"] not in pos:
                runner.add_request(e["id"])
                pos[e["id"]] = 0
            items.append(StepItem(e["id"], e["tokens"], e["want"]))
        logits = runner.step(items).float().cpu()
        runner.check_errors()
        r = 0
        for e in st["entries"]:
            for w in e["want"]:
                out[(e["id"], pos[e["id"]] + w)] = logits[r]
                r += 1
            pos[e["id"]] += len(e["tokens"])
        for rid in st["end"]:
            runner.free_request(rid)
            del pos[rid]
        runner.cache.check_consistent()
    return out
