"""Writes tests/golden/plain_tiny.json: a few logits of the plain implementation on the
tiny random models, so that an accidental change of the oracle itself is noticed.

The numbers come from the plain implementation alone (float64 on the CPU).  The
reference's model code cannot be run as a whole (TypeScript for Bun over CUDA kernels);
numbers from its kernels, part by part, are made by make_reference_kernel_golden.py.

    python tests/golden/make_golden.py
"""
import json
import os
import sys
import tempfile

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.join(os.path.dirname(HERE), "plain"))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import helpers as H          # noqa: E402
import qwen3_plain as P      # noqa: E402

out = {}
with tempfile.TemporaryDirectory() as tmp:
    for which in ("A", "B", "W"):
        d = H.make_model_dir(tmp, which)
        raw, w = H.read_model_dir(d)
        toks = H.random_tokens(37, raw["vocab_size"], 99)
        lg = P.forward(raw, w, toks, torch.float64)
        out[which] = {"tokens": toks, "last_logits_first8": lg[-1, :8].tolist(),
                      "argmax": int(lg[-1].argmax())}
with open(os.path.join(HERE, "plain_tiny.json"), "w") as f:
    json.dump(out, f, indent=1)
print("written")
