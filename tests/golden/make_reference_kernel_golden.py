#!/usr/bin/env python3
"""Numbers from bwasti/binfer's own CUDA kernels, for the plain implementation to be held to.

The reference's model code cannot be imported or compiled on a CPU (TypeScript for Bun
over CUDA kernels), but the kernels that hold its formulas are plain CUDA without any
instruction of one architecture: cuda/kernels/bf16_kernels.cu and
cuda/kernels/paged_attention.cu.  This script compiles those two files, unmodified, for
sm_100a (with one line of its own: ``binfer_get_current_stream``, which the reference
defines beside its cuBLAS wrapper, cuda/kernels/gemm.cu:40, and which here returns the
default stream), runs them on small inputs on a GPU and writes inputs and outputs to
``reference_kernels.npz`` beside this file.  ``tests/test_plain_against_reference_kernels.py``
then checks every part of the plain implementation against them, on any machine.

    python tests/golden/make_reference_kernel_golden.py [--reference DIR] [--out FILE]

``DIR`` holds the reference's ``cuda/`` folder (default: ``baseline/_ref`` in this
repository, an unmodified copy).  bfloat16 arrays are stored as their 16 bits (uint16).

Entry points called (file:line in the reference): binfer_rmsnorm_bf16
(bf16_kernels.cu:87), binfer_rotary_embedding_bf16 (:187), binfer_rotary_embedding_decode_bf16
(:388), binfer_swiglu_bf16 (:479), binfer_add_bf16 (:519), binfer_embedding_bf16 (:731),
binfer_compute_rope_cache_bf16 (:784), binfer_flash_attention_bf16 (:1007),
binfer_argmax_bf16 (:1334), binfer_paged_attention_bf16 (paged_attention.cu:491),
binfer_paged_kv_cache_update_bf16 (:612).  Every block id and token id given to them is in
range, and every context holds at least one token.
"""
import argparse
import ctypes
import math
import os
import subprocess
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
BLOCK = 16                     # the reference's page size (paged_attention.cu:16)


def build(reference_dir: str, out_dir: str) -> str:
    """Compile the reference's two kernel files for sm_100a into a shared library."""
    cuda = os.path.join(reference_dir, "cuda")
    srcs = [os.path.join(cuda, "kernels", f) for f in ("bf16_kernels.cu", "paged_attention.cu")]
    for s in srcs:
        if not os.path.exists(s):
            raise FileNotFoundError(s)
    shim = os.path.join(out_dir, "current_stream.cu")
    with open(shim, "w") as f:
        f.write('extern "C" void* binfer_get_current_stream() { return 0; }\n')
    lib = os.path.join(out_dir, "libbinfer_reference_kernels.so")
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-shared", "-Xcompiler",
           "-fPIC", "-I", os.path.join(cuda, "include"), *srcs, shim, "-o", lib]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed on the reference's kernels:\n" + r.stderr[-2000:])
    return lib


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def inputs() -> dict:
    """Every case's inputs, seeded; bfloat16 tensors on the CPU (int32 for ids and tables)."""
    g = torch.Generator().manual_seed(20240607)
    bf = torch.bfloat16

    def rn(*shape, scale=1.0):
        return (torch.randn(*shape, generator=g) * scale).to(bf)

    c = {}
    c["norm_x"], c["norm_w"] = rn(5, 96, scale=2.0), (1 + 0.1 * torch.randn(96, generator=g)).to(bf)
    c["norm_x"][4] = (c["norm_x"][4].float() * 0.002).to(bf)   # mean square near eps: eps shows
    # the head norms: a row is one head of one token (6 heads of 32 for 4 tokens)
    c["hnorm_x"], c["hnorm_w"] = rn(24, 32), (1 + 0.1 * torch.randn(32, generator=g)).to(bf)
    # rotation of a 7-token portion that starts at position 3: 3 query heads, 1 kv head of 32
    c["rope_q"], c["rope_k"] = rn(1, 7, 3, 32), rn(1, 7, 1, 32)
    # ... and of single tokens at positions of their own
    c["roped_q"], c["roped_k"] = rn(3, 3, 32), rn(3, 1, 32)
    c["roped_pos"] = torch.tensor([5, 0, 11], dtype=torch.int32)
    c["gate"], c["up"] = rn(2, 40, scale=3.0), rn(2, 40)
    c["add_a"], c["add_b"] = rn(3, 33), rn(3, 33)
    c["emb_table"] = rn(10, 24)
    c["emb_ids"] = torch.tensor([[3, 9, 0, 3]], dtype=torch.int32)
    # causal attention over 24 tokens: 4 query heads, 2 kv heads of 64
    c["att_q"], c["att_k"], c["att_v"] = rn(1, 24, 4, 64), rn(1, 24, 2, 64), rn(1, 24, 2, 64)
    # one far key that stands out for the last query (a lost or misplaced key shows)
    c["att_k"][0, 2] = 0
    c["att_k"][0, 2, :, 0] = 16.0
    c["att_q"][0, 23, :, 0] = 8.0
    c["att_v"][0, 2] = 4.0
    # paged attention: three sequences of 1, 17 and 40 keys in shuffled 16-token blocks
    c["pg_lens"] = torch.tensor([1, 17, 40], dtype=torch.int32)
    c["pg_tables"] = torch.tensor([[5, 0, 0], [2, 7, 0], [6, 1, 4]], dtype=torch.int32)
    c["pg_q"] = rn(3, 4, 64)
    c["pg_k"], c["pg_v"] = rn(8, BLOCK, 2, 64), rn(8, BLOCK, 2, 64)
    # cache write: two new tokens per sequence behind contexts of 15 and 3
    c["wr_lens"] = torch.tensor([15, 3], dtype=torch.int32)
    c["wr_tables"] = torch.tensor([[3, 1], [2, 0]], dtype=torch.int32)
    c["wr_k"], c["wr_v"] = rn(2, 2, 2, 64), rn(2, 2, 2, 64)
    c["logits"] = rn(3, 301, scale=4.0)
    for r in range(3):                       # no ties: the reference defines no winner among equals
        row = c["logits"][r].float()
        row[(7 * r + 123) % 301] = row.max() + 1.0
        c["logits"][r] = row.to(bf)
    return c


def rope_table(max_pos: int, head_dim: int, theta: float):
    """cos and sin [max_pos, head_dim / 2] as the engine's start-up builds them
    (src/engine/tp_context.ts:196-212): frequencies 1 / theta^(2i/d) rounded to float32,
    angles and functions in double, stored as float32; then to the kernels' bfloat16 by
    rounding (the reference truncates, src/tensor/tensor.ts:136-145)."""
    half = head_dim // 2
    freqs = np.array([1.0 / math.pow(theta, (2 * i) / head_dim) for i in range(half)],
                     dtype=np.float32).astype(np.float64)
    ang = np.arange(max_pos, dtype=np.float64)[:, None] * freqs[None, :]
    cos = torch.from_numpy(np.cos(ang).astype(np.float32)).to(torch.bfloat16)
    sin = torch.from_numpy(np.sin(ang).astype(np.float32)).to(torch.bfloat16)
    return cos, sin


def run_cases(lib_path: str, dev: str = "cuda:0") -> dict:
    """Run every case through the reference's kernels; inputs and outputs as numpy arrays."""
    lib = ctypes.CDLL(lib_path)
    c = inputs()
    d = {k: v.to(dev) for k, v in c.items()}
    out = {}

    def ok(code, what):
        torch.cuda.synchronize()
        if code != 0:
            raise RuntimeError(f"{what} returned {code}")

    i32, f32 = ctypes.c_int, ctypes.c_float
    # RMSNorm over rows, eps 1e-5; the head norms are the same kernel over (token, head) rows
    for name, eps in (("norm", 1e-5), ("hnorm", 1e-6)):
        x, w = d[name + "_x"], d[name + "_w"]
        y = torch.empty_like(x)
        ok(lib.binfer_rmsnorm_bf16(_p(x), _p(w), _p(y), i32(1), i32(x.shape[0]), i32(x.shape[1]),
                                   f32(eps)), "rmsnorm")
        out[name + "_y"] = y
    cos, sin = rope_table(16, 32, 10000.0)
    out["rope_cos"], out["rope_sin"] = cos, sin
    cosd, sind = cos.to(dev), sin.to(dev)
    q, k = d["rope_q"].clone(), d["rope_k"].clone()
    ok(lib.binfer_rotary_embedding_bf16(_p(q), _p(k), _p(cosd), _p(sind), i32(1), i32(7), i32(3),
                                        i32(1), i32(32), i32(3)), "rotary_embedding")
    out["rope_q_out"], out["rope_k_out"] = q, k
    q, k = d["roped_q"].clone(), d["roped_k"].clone()
    ok(lib.binfer_rotary_embedding_decode_bf16(_p(q), _p(k), _p(cosd), _p(sind),
                                               _p(d["roped_pos"]), i32(3), i32(3), i32(1),
                                               i32(32)), "rotary_embedding_decode")
    out["roped_q_out"], out["roped_k_out"] = q, k
    # the table as the reference's own kernel computes it (theta 1e4, no scaling)
    tc = torch.empty(16, 16, dtype=torch.bfloat16, device=dev)
    ts = torch.empty_like(tc)
    ok(lib.binfer_compute_rope_cache_bf16(_p(tc), _p(ts), i32(16), i32(32), f32(10000.0),
                                          f32(1.0)), "compute_rope_cache")
    out["table_cos"], out["table_sin"] = tc, ts
    y = torch.empty_like(d["gate"])
    ok(lib.binfer_swiglu_bf16(_p(d["gate"]), _p(d["up"]), _p(y),
                              ctypes.c_size_t(y.numel())), "swiglu")
    out["swiglu_y"] = y
    y = torch.empty_like(d["add_a"])
    ok(lib.binfer_add_bf16(_p(d["add_a"]), _p(d["add_b"]), _p(y), ctypes.c_size_t(y.numel())),
       "add")
    out["add_y"] = y
    y = torch.empty(1, 4, 24, dtype=torch.bfloat16, device=dev)
    ok(lib.binfer_embedding_bf16(_p(d["emb_table"]), _p(d["emb_ids"]), _p(y), i32(1), i32(4),
                                 i32(10), i32(24)), "embedding")
    out["emb_y"] = y
    # causal attention, whole, then only the last five queries with their offset
    scale = 1.0 / math.sqrt(64)
    o = torch.empty_like(d["att_q"])
    ok(lib.binfer_flash_attention_bf16(_p(d["att_q"]), _p(d["att_k"]), _p(d["att_v"]), _p(o),
                                       i32(1), i32(24), i32(24), i32(24), i32(0), i32(4), i32(2),
                                       i32(64), f32(scale), ctypes.c_bool(True)), "flash_attention")
    out["att_o"] = o
    q5 = d["att_q"][:, 19:].contiguous()
    o5 = torch.empty_like(q5)
    ok(lib.binfer_flash_attention_bf16(_p(q5), _p(d["att_k"]), _p(d["att_v"]), _p(o5), i32(1),
                                       i32(5), i32(24), i32(24), i32(19), i32(4), i32(2), i32(64),
                                       f32(scale), ctypes.c_bool(True)), "flash_attention+offset")
    out["att_o_last5"] = o5
    # paged attention (block tables and lengths are host pointers there)
    o = torch.empty_like(d["pg_q"])
    tables, lens = c["pg_tables"].contiguous(), c["pg_lens"].contiguous()
    ok(lib.binfer_paged_attention_bf16(_p(d["pg_q"]), _p(d["pg_k"]), _p(d["pg_v"]), _p(o),
                                       _p(tables), _p(lens), i32(3), i32(4), i32(2), i32(64),
                                       i32(BLOCK), i32(3), f32(scale)), "paged_attention")
    out["pg_o"] = o
    kc = torch.zeros(4, BLOCK, 2, 64, dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)
    tables, lens = c["wr_tables"].contiguous(), c["wr_lens"].contiguous()
    ok(lib.binfer_paged_kv_cache_update_bf16(_p(kc), _p(vc), _p(d["wr_k"]), _p(d["wr_v"]),
                                             _p(tables), _p(lens), i32(2), i32(2), i32(2), i32(64),
                                             i32(2)), "paged_kv_cache_update")
    out["wr_kc"], out["wr_vc"] = kc, vc
    ids = torch.empty(3, dtype=torch.int32, device=dev)
    ok(lib.binfer_argmax_bf16(_p(d["logits"]), _p(ids), i32(3), i32(301)), "argmax")
    out["argmax_ids"] = ids

    arrays = {}
    for k, v in {**c, **out}.items():
        arrays[k] = _bits(v) if v.dtype == torch.bfloat16 else v.cpu().numpy()
    return arrays


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.path.join(ROOT, "baseline", "_ref"))
    ap.add_argument("--out", default=os.path.join(HERE, "reference_kernels.npz"))
    args = ap.parse_args()
    with tempfile.TemporaryDirectory() as tmp:
        lib = build(args.reference, tmp)
        arrays = run_cases(lib)
    np.savez_compressed(args.out, **arrays)
    print(f"wrote {args.out}: {len(arrays)} arrays, {os.path.getsize(args.out)} bytes")


if __name__ == "__main__":
    sys.exit(main())
