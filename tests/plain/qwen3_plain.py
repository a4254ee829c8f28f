"""A plain, slow Qwen3 dense decoder: whole sequences, no cache, one function per part.

This is the tests' oracle.  It shares no code with ``binfer_b200``: it reads the
raw config.json dictionary and a name -> tensor dictionary itself, and runs on
the CPU with ordinary tensor arithmetic.

Nothing of bwasti/binfer's model code can be imported or compiled on a CPU: it is
TypeScript for Bun (``bun:ffi``) over CUDA kernels and cuBLAS.  So each function
restates the reference's formulas and cites the file and lines it restates (paths
inside the bwasti/binfer project).  The parts are also held to the reference's
execution: its kernel files compile unmodified for sm_100a, and what they made of
small inputs on a B200 is committed under ``tests/golden/`` with the script that
ran them; ``tests/test_plain_against_reference_kernels.py`` compares every part
here with those numbers.

``dtype`` is the working precision (float32 by default; float64 gives an oracle
whose own rounding is negligible).  Rotation angles are always formed in
float32, as the engine forms them.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch


# ------------------------------------------------------------------ configuration
def read_config(raw: dict) -> dict:
    """Sizes and constants with the reference's defaults (src/model/config.ts:73-192)."""
    h = raw["hidden_size"]
    heads = raw["num_attention_heads"]
    c = {
        "hidden": h,
        "heads": heads,
        "kv_heads": raw.get("num_key_value_heads") or heads,          # config.ts:108-112
        "head_dim": raw.get("head_dim") or h // heads,                # config.ts:115-119
        "inter": raw["intermediate_size"],
        "layers": raw["num_hidden_layers"],
        "vocab": raw["vocab_size"],
        "eps": raw.get("rms_norm_eps", 1e-5),                         # config.ts:161
        "theta": raw.get("rope_theta", 10000.0),                      # config.ts:163
        "tied": raw.get("tie_word_embeddings", False),                # config.ts:168
        "factor": 1.0,
    }
    sc = raw.get("rope_scaling")
    if sc and sc.get("rope_type", sc.get("type")) == "linear":
        c["factor"] = float(sc["factor"])
    # windows only with use_sliding_window; then layer_types wins, else layers from
    # max_window_layers on are windowed
    n, w = c["layers"], raw.get("sliding_window")
    if not raw.get("use_sliding_window"):
        c["windows"] = [None] * n
    elif raw.get("layer_types"):
        c["windows"] = [w if t == "sliding_attention" else None for t in raw["layer_types"]]
    elif raw.get("use_sliding_window") and w:
        first = raw.get("max_window_layers") or 0
        c["windows"] = [w if i >= first else None for i in range(n)]
    else:
        c["windows"] = [None] * n
    return c


# A model of the reference's bfloat16 arithmetic, for error bounds: every function below
# computes in the working precision; ``_r(x, rt)`` then rounds a result to ``rt`` (bfloat16)
# wherever the reference's kernels store one in bfloat16 (with ``rt`` None, nowhere).
def _r(x: torch.Tensor, rt: Optional[torch.dtype]) -> torch.Tensor:
    return x if rt is None else x.to(rt).to(x.dtype)


# ------------------------------------------------------------------------- parts
def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """x[t,:] = E[ids[t],:], no scaling (cuda/kernels/bf16_kernels.cu:711-729)."""
    return table[ids.long()]


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w over the last axis; the weight multiplies
    directly, no ``1 + w`` (cuda/kernels/bf16_kernels.cu:40-84)."""
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(ms + eps) * w


def rope_angles(positions: torch.Tensor, rotary_dim: int, theta: float,
                factor: float = 1.0) -> torch.Tensor:
    """a[p, i] = p * theta^(-2i/d) for i < d/2 (src/engine/tp_context.ts:181-221);
    the frequency is rounded to float32 and the product is formed in float32."""
    i = torch.arange(rotary_dim // 2, dtype=torch.float64)
    inv_freq = (float(theta) ** (-2.0 * i / rotary_dim) / factor).to(torch.float32)
    return positions.to(torch.float32)[:, None] * inv_freq[None, :]


def apply_rope(x: torch.Tensor, angles: torch.Tensor) -> torch.Tensor:
    """Rotate-half layout on ``x [T, heads, d]``: pairs (i, i + d/2)
    (cuda/kernels/bf16_kernels.cu:133-185): x'[i] = x[i] cos a - x[i+d/2] sin a,
    x'[i+d/2] = x[i] sin a + x[i+d/2] cos a.  Dimensions past 2 * angles.shape[1]
    pass through."""
    half = angles.shape[1]
    cos = torch.cos(angles.to(torch.float64)).to(x.dtype)[:, None, :]
    sin = torch.sin(angles.to(torch.float64)).to(x.dtype)[:, None, :]
    x1, x2, rest = x[..., :half], x[..., half:2 * half], x[..., 2 * half:]
    return torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos, rest], dim=-1)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                     window: Optional[int] = None) -> torch.Tensor:
    """softmax(q k^T * scale) v with keys j <= p, query head h reading kv head
    h // (heads / kv_heads) (cuda/kernels/bf16_kernels.cu:909-973;
    cuda/kernels/paged_attention.cu:408-487).  ``window``: only keys j > p - window.
    Shapes: q [T, heads, d], k and v [T, kv_heads, d] -> [T, heads, d]."""
    T, heads, d = q.shape
    group = heads // k.shape[1]
    out = torch.empty_like(q)
    p = torch.arange(T)
    allowed = p[None, :] <= p[:, None]
    if window is not None:
        allowed &= p[None, :] > p[:, None] - window
    for h in range(heads):
        g = h // group
        s = (q[:, h, :] @ k[:, g, :].T) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        out[:, h, :] = torch.softmax(s, dim=-1) @ v[:, g, :]
    return out


def attention_block(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, c: dict,
                    positions: torch.Tensor, window: Optional[int],
                    rt: Optional[torch.dtype] = None) -> torch.Tensor:
    """q,k,v projections, per-head RMSNorm of q and k with the layer norms' eps, then
    the rotation, attention and the output projection
    (src/engine/batched_engine.ts:811-839,861-876,1061-1090,1116-1118)."""
    T = x.shape[0]
    nh, nkv, d = c["heads"], c["kv_heads"], c["head_dim"]
    q = _r(x @ w[prefix + "q_proj.weight"].T, rt).view(T, nh, d)
    k = _r(x @ w[prefix + "k_proj.weight"].T, rt).view(T, nkv, d)
    v = _r(x @ w[prefix + "v_proj.weight"].T, rt).view(T, nkv, d)
    q = _r(rms_norm(q, w[prefix + "q_norm.weight"], c["eps"]), rt)
    k = _r(rms_norm(k, w[prefix + "k_norm.weight"], c["eps"]), rt)
    ang = rope_angles(positions, d, c["theta"], c["factor"])
    q, k = _r(apply_rope(q, ang), rt), _r(apply_rope(k, ang), rt)
    a = _r(causal_attention(q, k, v, 1.0 / math.sqrt(d), window), rt)   # batched_engine.ts:1062
    return _r(a.reshape(T, nh * d) @ w[prefix + "o_proj.weight"].T, rt)


def silu_mul(g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """silu(g) * u with silu(g) = g / (1 + exp(-g)) (cuda/kernels/bf16_kernels.cu:461-477)."""
    return (g / (1.0 + torch.exp(-g))) * u


def swiglu_mlp(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str,
               rt: Optional[torch.dtype] = None) -> torch.Tensor:
    """down( silu(gate(x)) * up(x) ) (src/engine/batched_engine.ts:1243-1265)."""
    g = _r(x @ w[prefix + "gate_proj.weight"].T, rt)
    u = _r(x @ w[prefix + "up_proj.weight"].T, rt)
    return _r(_r(silu_mul(g, u), rt) @ w[prefix + "down_proj.weight"].T, rt)


def decoder_layer(x: torch.Tensor, w: Dict[str, torch.Tensor], i: int, c: dict,
                  positions: torch.Tensor, rt: Optional[torch.dtype] = None) -> torch.Tensor:
    """Pre-norm residual block: x + attn(norm(x)), then x + mlp(norm(x))
    (src/engine/batched_engine.ts:800-1314; the sums are formed in float and stored in
    the activations' type, cuda/kernels/bf16_kernels.cu:504-517)."""
    p = f"model.layers.{i}."
    n = _r(rms_norm(x, w[p + "input_layernorm.weight"], c["eps"]), rt)
    x = _r(x + attention_block(n, w, p + "self_attn.", c, positions, c["windows"][i], rt), rt)
    n = _r(rms_norm(x, w[p + "post_attention_layernorm.weight"], c["eps"]), rt)
    return _r(x + swiglu_mlp(n, w, p + "mlp.", rt), rt)


def forward(raw_config: dict, weights: Dict[str, torch.Tensor], ids: Sequence[int],
            dtype: torch.dtype = torch.float32,
            rows: Optional[Sequence[int]] = None,
            round_to: Optional[torch.dtype] = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` at every position of one whole sequence
    (final norm and head: src/engine/batched_engine.ts:1733-1770; the head is the
    embedding table when ``tie_word_embeddings``, :1753-1755).  ``rows``: only these
    positions' logits (the layers still run the whole sequence).  ``round_to``
    (bfloat16): every result that the reference stores in bfloat16, the logits
    included (:2609), is rounded to it: a model of the reference's own rounding,
    against which the engine's bfloat16 error can be held."""
    c = read_config(raw_config)
    w = {k: t.to(dtype) for k, t in weights.items()}
    ids_t = torch.as_tensor(list(ids), dtype=torch.long)
    positions = torch.arange(len(ids_t))
    x = embedding(ids_t, w["model.embed_tokens.weight"])
    for i in range(c["layers"]):
        x = decoder_layer(x, w, i, c, positions, round_to)
    if rows is not None:
        x = x[torch.as_tensor(list(rows), dtype=torch.long)]
    x = _r(rms_norm(x, w["model.norm.weight"], c["eps"]), round_to)
    head = w["model.embed_tokens.weight"] if c["tied"] else w["lm_head.weight"]
    return _r(x @ head.T, round_to)


# ---------------------------------------------------------------------- sampling
def sample(logits: torch.Tensor, temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0,
           repetition_penalty: float = 1.0, generated: Sequence[int] = (),
           uniform: float = 0.0) -> int:
    """One token from one row of logits, in the reference's order of operations
    (src/engine/sampler.ts:57-157): repetition penalty (s > 0 ? s / pen : s * pen)
    on every generated token, argmax if the temperature is 0 (first maximal
    index, :171-181), else divide by the temperature, keep the top_k largest,
    cut at the first prefix of descending probabilities whose sum reaches top_p,
    renormalise and draw.  The draw walks the kept tokens in index order and
    returns the first whose running sum exceeds ``uniform``."""
    s = logits.to(torch.float64).clone()
    if repetition_penalty != 1.0:
        for t in generated:                 # once per occurrence (sampler.ts:64-73)
            s[t] = s[t] / repetition_penalty if s[t] > 0 else s[t] * repetition_penalty
    if temperature == 0:
        return int(torch.argmax(s))          # torch returns the first maximal index
    s = s / temperature
    order = torch.argsort(s, descending=True, stable=True)
    cutoff = len(s)
    if 0 < top_k < cutoff:
        cutoff = top_k
    if top_p < 1.0:
        p = torch.softmax(s[order[:cutoff]], dim=0)
        cum = torch.cumsum(p, dim=0)
        cutoff = int((cum >= top_p).nonzero()[0]) + 1 if bool((cum >= top_p).any()) else cutoff
    keep = torch.zeros(len(s), dtype=torch.bool)
    keep[order[:cutoff]] = True
    p = torch.softmax(s.masked_fill(~keep, float("-inf")), dim=0)
    cum = torch.cumsum(p, dim=0)
    hit = (cum > uniform) & keep
    if bool(hit.any()):
        return int(hit.nonzero()[0])
    return int(keep.nonzero()[-1])


def greedy_generate(raw_config: dict, weights: Dict[str, torch.Tensor], prompt: Sequence[int],
                    max_tokens: int, eos: Sequence[int] = (),
                    dtype: torch.dtype = torch.float32) -> List[int]:
    """Recompute the whole sequence for every new token; the stop token is kept in
    the output (src/engine/batched_engine.ts:3157-3168)."""
    ids, out = list(prompt), []
    for _ in range(max_tokens):
        tok = int(torch.argmax(forward(raw_config, weights, ids, dtype)[-1]))
        out.append(tok)
        ids.append(tok)
        if tok in eos:
            break
    return out
