"""The plain implementation against numbers that bwasti/binfer's own CUDA kernels produced.

``tests/golden/reference_kernels.npz`` holds small inputs and what the reference's kernels
(cuda/kernels/bf16_kernels.cu, cuda/kernels/paged_attention.cu, compiled unmodified for
sm_100a and run on a B200 by ``tests/golden/make_reference_kernel_golden.py``) made of them.
Each part of the plain implementation is run on the same inputs in float64 and has to agree
within the rounding of the kernels' bfloat16 outputs, so that the plain implementation
rests on the reference's execution, not only on a reading of its source: the norm's weight
multiplies directly and eps sits inside the root; the rotation pairs (i, i + d/2) at the
token's absolute position; query head h reads kv head h // (heads / kv_heads); scores are
scaled by 1/sqrt(d) and a query at p sees keys j <= p; silu(g) = g / (1 + exp(-g)); a key
at position p lives in block table[p // 16], slot p % 16.
"""
import math
import os

import numpy as np
import pytest
import torch

import qwen3_plain as P

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_kernels.npz")
BLOCK = 16

# a bfloat16 result is within half a unit in the last place (2^-9 of its magnitude) of the
# float result it was rounded from; three of those, relative to the tensor's largest value
TOL = 3 * 2.0 ** -9


def _load():
    z = np.load(GOLDEN)

    def get(name):
        a = z[name]
        if a.dtype == np.uint16:                     # bfloat16, stored as its bits
            return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16).double()
        return torch.from_numpy(a.copy())
    return get


@pytest.fixture(scope="module")
def ref():
    assert os.path.exists(GOLDEN), "tests/golden/reference_kernels.npz is missing"
    return _load()


def _close(plain, got, tol=TOL):
    err = float((plain - got).abs().max())
    assert err <= tol * float(plain.abs().max()), f"differs by {err:.4g} of {float(plain.abs().max()):.4g}"


def test_rms_norm(ref):
    _close(P.rms_norm(ref("norm_x"), ref("norm_w"), 1e-5), ref("norm_y"))
    # the row whose mean square is about eps: eps inside the root, not outside, not absent
    x, y = ref("norm_x")[4], ref("norm_y")[4]
    _close(P.rms_norm(x, ref("norm_w"), 1e-5), y)
    no_eps = P.rms_norm(x, ref("norm_w"), 0.0)
    assert float((no_eps - y).abs().max()) > 20 * TOL * float(y.abs().max())
    # the head norms: the same formula over the elements of one head
    _close(P.rms_norm(ref("hnorm_x"), ref("hnorm_w"), 1e-6), ref("hnorm_y"))


def test_rope_table_and_rotation(ref):
    pos = torch.arange(16)
    ang = P.rope_angles(pos, 32, 10000.0)
    # the table the reference's own kernel computes (cosf / sinf of float angles)
    _close(torch.cos(ang.double()), ref("table_cos"))
    _close(torch.sin(ang.double()), ref("table_sin"))
    # rotation of a portion that starts at position 3; the kernels read a bfloat16 table, so
    # the angles' functions carry that rounding too (two more half units)
    tol = 5 * 2.0 ** -9
    ang = P.rope_angles(torch.arange(3, 10), 32, 10000.0)
    _close(P.apply_rope(ref("rope_q")[0], ang), ref("rope_q_out")[0], tol)
    _close(P.apply_rope(ref("rope_k")[0], ang), ref("rope_k_out")[0], tol)
    ang = P.rope_angles(ref("roped_pos"), 32, 10000.0)
    _close(P.apply_rope(ref("roped_q"), ang), ref("roped_q_out"), tol)
    _close(P.apply_rope(ref("roped_k"), ang), ref("roped_k_out"), tol)
    # the other pairing in use elsewhere, (2i, 2i + 1), is far from what the kernels did
    x, want = ref("rope_q")[0], ref("rope_q_out")[0]
    ang = P.rope_angles(torch.arange(3, 10), 32, 10000.0).double()
    c, sn = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    other = torch.empty_like(x)
    other[..., 0::2] = x[..., 0::2] * c - x[..., 1::2] * sn
    other[..., 1::2] = x[..., 0::2] * sn + x[..., 1::2] * c
    assert float((other - want).abs().max()) > 0.5


def test_silu_mul_add_embedding_argmax(ref):
    _close(P.silu_mul(ref("gate"), ref("up")), ref("swiglu_y"))
    _close(ref("add_a") + ref("add_b"), ref("add_y"))
    got = P.embedding(ref("emb_ids")[0], ref("emb_table"))
    assert torch.equal(got, ref("emb_y")[0])
    ids = [P.sample(row, temperature=0.0) for row in ref("logits")]
    assert ids == ref("argmax_ids").tolist()


def test_causal_attention(ref):
    q, k, v = ref("att_q")[0], ref("att_k")[0], ref("att_v")[0]
    out = P.causal_attention(q, k, v, 1.0 / math.sqrt(64))
    _close(out, ref("att_o")[0])
    # the far key that stands out carries the last query's output
    assert float(ref("att_o")[0][23].mean()) > 3.0
    # queries at an offset see the keys up to their absolute position
    _close(out[19:], ref("att_o_last5")[0])


def test_paged_attention_and_cache_write(ref):
    lens, tables = ref("pg_lens").tolist(), ref("pg_tables").tolist()
    kc, vc, q = ref("pg_k"), ref("pg_v"), ref("pg_q")
    for s, n in enumerate(lens):
        # key p of a sequence: block table[p // 16], slot p % 16 (cuda/kernels/paged_attention.cu:408-416)
        k = torch.stack([kc[tables[s][p // BLOCK], p % BLOCK] for p in range(n)])
        v = torch.stack([vc[tables[s][p // BLOCK], p % BLOCK] for p in range(n)])
        qs = torch.zeros(n, 4, 64, dtype=torch.float64)
        qs[-1] = q[s]
        out = P.causal_attention(qs, k, v, 1.0 / math.sqrt(64))[-1]
        _close(out, ref("pg_o")[s])
    # the write: token t of sequence s goes to position lens[s] + t
    lens, tables = ref("wr_lens").tolist(), ref("wr_tables").tolist()
    want_k = torch.zeros(4, BLOCK, 2, 64, dtype=torch.float64)
    want_v = torch.zeros_like(want_k)
    for s in range(2):
        for t in range(2):
            p = lens[s] + t
            want_k[tables[s][p // BLOCK], p % BLOCK] = ref("wr_k")[s, t]
            want_v[tables[s][p // BLOCK], p % BLOCK] = ref("wr_v")[s, t]
    assert torch.equal(want_k, ref("wr_kc")) and torch.equal(want_v, ref("wr_vc"))
