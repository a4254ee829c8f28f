"""bin/trace_run as a user runs it: JSON steps on standard input, <step>.f32 files out."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers as H
import qwen3_plain as P

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _replay(model_dir, dtype, steps, out_dir, max_tokens):
    """Feed the steps one at a time, each only after the last one's ``done`` line."""
    proc = subprocess.Popen(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir,
         "--dtype", dtype, "--out", out_dir, "--max-tokens", str(max_tokens)],
        stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        for st in steps:
            proc.stdin.write(json.dumps(st) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {st['step']}", f"expected 'done {st['step']}', got {line!r}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()


def _collect(steps, out_dir, vocab):
    got, pos = {}, {}
    for st in steps:
        wanted = sum(len(e["want"]) for e in st["entries"])
        path = os.path.join(out_dir, f"{st['step']}.f32")
        if wanted == 0:
            assert not os.path.exists(path)
        else:
            arr = np.fromfile(path, dtype="<f4").reshape(wanted, vocab)
            r = 0
            for e in st["entries"]:
                for w in e["want"]:
                    got[(e["id"], pos.get(e["id"], 0) + w)] = torch.from_numpy(arr[r].copy())
                    r += 1
        for e in st["entries"]:
            pos[e["id"]] = pos.get(e["id"], 0) + len(e["tokens"])
        for rid in st["end"]:
            pos.pop(rid, None)
    return got


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 3e-2)])
def test_trace_run_mixed_trace_with_page_reuse(cuda_device, tmp_path, dtype, tol):
    which = "B"
    tdtype = torch.float32 if dtype == "float32" else torch.bfloat16
    d = H.make_model_dir(tmp_path, which, tdtype)
    raw, w = H.read_model_dir(d)
    vocab = raw["vocab_size"]
    reqs = {f"r{i}": H.random_tokens(n, vocab, 31 * i + n)
            for i, n in enumerate([70, 33, 90, 12, 64, 41])}
    steps = H.trace_mixed(reqs)
    # some steps want nothing, some only a few places
    for i, st in enumerate(steps):
        if i % 4 == 1:
            for e in st["entries"]:
                e["want"] = []
        elif i % 4 == 2:
            for e in st["entries"]:
                e["want"] = e["want"][-1:]
    # the most tokens live at a time, each request rounded up to a multiple of 64
    live, peak = {}, 0
    for st in steps:
        for e in st["entries"]:
            live[e["id"]] = live.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // 64) * 64 for n in live.values()))
        for rid in st["end"]:
            live.pop(rid)
    out_dir = str(tmp_path / f"out_{dtype}")
    _replay(d, dtype, steps, out_dir, peak)
    got = _collect(steps, out_dir, vocab)
    assert got
    ref = {rid: P.forward(raw, w, toks, torch.float64) for rid, toks in reqs.items()}
    worst = max(H.rel_err(row, ref[rid][p]) for (rid, p), row in got.items())
    assert worst <= tol, f"worst relative error {worst:.3g}"


def test_trace_run_refuses_a_broken_model_folder(cuda_device, tmp_path):
    d = H.make_model_dir(tmp_path, "A")
    raw, w = H.read_model_dir(d)
    del w["model.norm.weight"]
    from binfer_b200.weights import save_file
    save_file(w, os.path.join(d, "model.safetensors"))
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d,
                        "--dtype", "float32", "--out", str(tmp_path / "o"), "--max-tokens", "64"],
                       input="", capture_output=True, text=True, timeout=120)
    assert r.returncode != 0
    assert "missing tensors (1): model.norm.weight" in r.stderr
