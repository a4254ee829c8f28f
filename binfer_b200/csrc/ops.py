"""Python bindings of the CUDA library: one function per kernel launcher.

Tensors are passed as raw device pointers through ctypes, on torch's current
stream.  There is no fallback of any kind: if the library cannot be built or
loaded, or a tensor is not on a CUDA device, the call raises.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build

_lib = None
_launches = 0      # kernels of this library launched so far (for the bench's count)

_c_int, _c_ll, _c_float, _c_void_p = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p


class KernelError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """The loaded library; built on first use."""
    global _lib
    if _lib is None:
        path = build.ensure_built()
        try:
            _lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load the engine's CUDA library {path}: {e}") from None
    return _lib


def launches() -> int:
    return _launches


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"unsupported activation dtype {t.dtype} (float32 or bfloat16)")


def _ptr(t: Optional[torch.Tensor]) -> _c_void_p:
    if t is None:
        return _c_void_p(0)
    if not t.is_cuda:
        raise KernelError("the engine's kernels take CUDA tensors only (no CPU path)")
    return _c_void_p(t.data_ptr())


def _stream() -> _c_void_p:
    return _c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(code: int, what: str) -> None:
    global _launches
    _launches += 1
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code}")


_profiler = None   # an object with begin(name) / end(name), set by binfer_b200.profiling


def set_profiler(p) -> None:
    global _profiler
    _profiler = p


def _run(name: str, fn, *args) -> None:
    p = _profiler
    if p is not None:
        p.begin(name)
    code = fn(*args)
    if p is not None:
        p.end(name)
    _check(code, name)


def count_library_launch(name: str = "gemm") -> None:
    """A library matrix product was launched (counted apart from the engine's own kernels)."""
    global _library_launches
    _library_launches += 1


_library_launches = 0


def library_launches() -> int:
    return _library_launches


def _want(t: torch.Tensor, dtype: torch.dtype, name: str) -> None:
    if t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


# ------------------------------------------------------------------ elementwise
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float,
                 err: torch.Tensor) -> None:
    """out[t] = table[ids[t]] * scale; out is the float residual stream [T, H]."""
    _want(ids, torch.int32, "ids"); _want(out, torch.float32, "out")
    T, H = out.shape
    _run("embed_gather", lib().bf_embed_gather, _ptr(table), _c_int(_dtype_code(table)), _ptr(ids), _ptr(out),
                                 _c_int(T), _c_int(H), _c_int(table.shape[0]), _c_float(scale),
                                 _ptr(err), _stream())


def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                out: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None,
                write_back: bool = True) -> None:
    """out[i] = rmsnorm(resid[r] + delta[r]) * weight with r = rows[i] (or i); the
    sum is written back to resid when ``write_back``."""
    _want(resid, torch.float32, "resid"); _want(weight, torch.float32, "weight")
    n, H = out.shape
    if delta is not None and (delta.dtype != out.dtype or not delta.is_contiguous()):
        raise KernelError("delta must be contiguous and of the output's dtype")
    if rows is not None:
        _want(rows, torch.int32, "rows")
    _run("add_rmsnorm", lib().bf_add_rmsnorm, _ptr(resid), _ptr(delta), _ptr(weight), _ptr(out), _ptr(rows),
                                _c_int(n), _c_int(H), _c_float(eps), _c_int(_dtype_code(out)),
                                _c_int(1 if write_back else 0), _stream())


def residual_add(resid: torch.Tensor, delta: torch.Tensor) -> None:
    _want(resid, torch.float32, "resid")
    _run("residual_add", lib().bf_residual_add, _ptr(resid), _ptr(delta), _c_ll(resid.numel()),
                                 _c_int(_dtype_code(delta)), _stream())


class RowScale:
    """A factor per row that is still to be applied: ``rsqrt(partials[t].sum() / width + eps)``.

    It is what a product that also prepared the next norm (``gemm_bf16_cluster_add_norm``)
    leaves out, because no CTA of it sees a whole row.  A linear map commutes with the
    factor, so the kernel after the next product applies it (``qk_norm_rope_kv_write``,
    ``silu_mul``).  ``partials`` is float32 ``[rows, count]``, contiguous."""
    __slots__ = ("partials", "width", "eps")

    def __init__(self, partials: torch.Tensor, width: int, eps: float):
        self.partials, self.width, self.eps = partials, int(width), float(eps)

    def factors(self) -> torch.Tensor:
        """The factors themselves, float32 ``[rows]`` (for tests and for parts that cannot
        take a RowScale)."""
        return torch.rsqrt(self.partials.sum(dim=1) / self.width + self.eps)


def _row_scale_args(rs: Optional["RowScale"], rows: int):
    if rs is None:
        return _ptr(None), _c_int(0), _c_int(0), _c_float(0.0)
    p = rs.partials
    if p.dtype != torch.float32 or not p.is_contiguous() or p.dim() != 2 or p.shape[0] < rows:
        raise KernelError("row scale: partials must be contiguous float32 [rows, count]")
    return _ptr(p), _c_int(p.shape[1]), _c_int(rs.width), _c_float(rs.eps)


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor,
             row_scale: Optional[RowScale] = None) -> None:
    """out[t, c] = silu(f gate_up[t, c]) * f gate_up[t, I + c]; f = 1 without ``row_scale``
    (which is taken for bfloat16 and I a multiple of 8, at least 256)."""
    T, I = out.shape
    if gate_up.shape != (T, 2 * I) or not gate_up.is_contiguous() or gate_up.dtype != out.dtype:
        raise KernelError("silu_mul: gate_up must be contiguous [T, 2*I] of the output's dtype")
    if row_scale is not None:
        if out.dtype != torch.bfloat16 or I % 8 or I < 256:
            raise KernelError("silu_mul: a row scale needs bfloat16 and I % 8 == 0, I >= 256")
        _run("silu_mul_scaled", lib().bf_silu_mul_scaled, _ptr(gate_up), _ptr(out), _c_int(T),
             _c_int(I), *_row_scale_args(row_scale, T), _stream())
        return
    _run("silu_mul", lib().bf_silu_mul, _ptr(gate_up), _ptr(out), _c_int(T), _c_int(I),
                             _c_int(_dtype_code(out)), _stream())


def copy_ids(dst: torch.Tensor, src: torch.Tensor, pairs: torch.Tensor, n: int) -> None:
    """dst[pairs[i, 0]] = src[pairs[i, 1]] for i < n (int32 everywhere)."""
    _want(dst, torch.int32, "dst"); _want(src, torch.int32, "src"); _want(pairs, torch.int32, "pairs")
    _run("copy_ids", lib().bf_copy_ids, _ptr(dst), _ptr(src), _ptr(pairs), _c_int(n), _stream())


# ------------------------------------------------------------------- attention
def qk_norm_rope_kv_write(qkv: torch.Tensor, q_w: Optional[torch.Tensor],
                          k_w: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor],
                          positions: torch.Tensor, slots: Optional[torch.Tensor],
                          q_out: torch.Tensor, k_cache: Optional[torch.Tensor],
                          v_cache: Optional[torch.Tensor], nh: int, nkv: int, d: int,
                          eps: float, err: torch.Tensor,
                          row_scale: Optional[RowScale] = None) -> None:
    """Per-head RMSNorm of q and k, rotation, q to ``q_out [T, nh*d]``, k and v into
    cache pages ``[pages, nkv, page_size, d]`` at ``slots``.  With ``row_scale`` the rows of
    ``qkv`` are first multiplied by their factors."""
    T = qkv.shape[0]
    if qkv.stride(1) != 1:
        raise KernelError("qkv rows must be contiguous")
    rot_half = 0 if inv_freq is None else inv_freq.numel()
    page_size = k_cache.shape[2] if k_cache is not None else 1
    num_slots = k_cache.shape[0] * page_size if k_cache is not None else 0
    if k_cache is not None and not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise KernelError("cache pages must be contiguous")
    _run("qk_norm_rope_kv_write", lib().bf_qk_norm_rope_kv_write, 
        _ptr(qkv), _c_ll(qkv.stride(0)), _ptr(q_w), _ptr(k_w), _ptr(inv_freq), _c_int(rot_half),
        _ptr(positions), _ptr(slots), _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _c_int(T),
        _c_int(nh), _c_int(nkv if k_cache is not None else 0), _c_int(d), _c_int(page_size),
        _c_ll(num_slots), _c_float(eps), _c_int(_dtype_code(qkv)),
        *_row_scale_args(row_scale, T), _ptr(err), _stream())


def paged_attention_generic(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                            seq_of_token: torch.Tensor, positions: torch.Tensor,
                            block_tables: torch.Tensor, out: torch.Tensor, nh: int, nkv: int,
                            d: int, window: Optional[int], scale: float,
                            err: torch.Tensor, softcap: float = 0.0,
                            slopes: Optional[torch.Tensor] = None,
                            sinks: Optional[torch.Tensor] = None) -> None:
    """Attention of every token row over its request's pages, any sizes.  ``softcap``,
    ``slopes`` (float32 ``[nh]``) and ``sinks`` (float32 ``[nh]``) change the scores as
    ``config.specs.ScoreSpec`` says; by default nothing is changed."""
    T = q.shape[0]
    if d > 256:
        raise KernelError(f"attention: head_dim {d} is not supported (at most 256)")
    for name, t in (("slopes", slopes), ("sinks", sinks)):
        if t is not None:
            _want(t, torch.float32, name)
            if t.numel() != nh:
                raise KernelError(f"attention: {name} must have one entry per query head")
    _run("paged_attention_generic", lib().bf_paged_attention_generic, 
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(seq_of_token), _ptr(positions),
        _ptr(block_tables), _c_int(block_tables.stride(0)), _ptr(out), _c_int(T), _c_int(nh),
        _c_int(nkv), _c_int(d), _c_int(k_cache.shape[2]), _c_int(k_cache.shape[0]),
        _c_int(window or 0), _c_float(scale), _c_float(softcap), _ptr(slopes), _ptr(sinks),
        _c_int(_dtype_code(q)), _ptr(err), _stream())


DECODE_HEAD_DIMS = (32, 64, 96, 128, 256)
DECODE_SPLIT_KEYS = 128


def decode_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     rows: Optional[torch.Tensor], n_rows: int, seq_of_token: torch.Tensor,
                     positions: torch.Tensor, block_tables: torch.Tensor, out: torch.Tensor,
                     nh: int, nkv: int, d: int, window: Optional[int], scale: float,
                     max_ctx_len: int, err: torch.Tensor, variant: str = "auto",
                     scratch=None) -> None:
    """Split-KV attention for rows that bring one token each (bfloat16 only).

    ``rows`` lists the token rows to run (None: rows 0..n_rows-1); ``max_ctx_len``
    bounds the context of every such row (a row beyond it sets the error word's
    "splits" bit and loses its far keys; nothing is read or written past the scratch).
    Scratch for the splits' partial results is taken from torch's allocator, or given as
    ``scratch = (part_o [n_rows, nh, splits, d], part_ml [n_rows, nh, splits, 2])`` float32,
    whose ``splits`` then is the room there is.  ``variant``: ``persistent`` (resident CTAs that walk
    the work with a ring of TMA-fed tiles; head sizes 64/128/256, page sizes 8..128 that
    divide 128, at most 16 query heads per kv head and 512 rows), ``tma`` (one CTA per split,
    bulk tensor copies; the same head and page sizes), ``cp_async`` (every size in
    DECODE_HEAD_DIMS, any page size), or ``auto``: the first of these that applies."""
    if q.dtype != torch.bfloat16 or d not in DECODE_HEAD_DIMS:
        raise KernelError(f"decode_attention: bfloat16 and head_dim in {DECODE_HEAD_DIMS} only")
    if variant not in ("auto", "persistent", "tma", "cp_async"):
        raise KernelError(f"decode_attention: unknown variant {variant!r}")
    page_size = k_cache.shape[2]
    tma_ok = d in (64, 128, 256) and 8 <= page_size <= 128 and 128 % page_size == 0
    persistent_ok = (tma_ok and nh // nkv <= 16 and n_rows <= 512 and q.is_contiguous()
                     and q.data_ptr() % 16 == 0)
    if variant == "tma" and not tma_ok:
        raise KernelError(f"decode_attention: the tma variant does not take head_dim {d} with "
                          f"pages of {page_size}")
    if variant == "persistent" and not persistent_ok:
        raise KernelError(f"decode_attention: the persistent variant does not take head_dim {d}, "
                          f"pages of {page_size}, {nh // nkv} heads per kv head, {n_rows} rows")
    if persistent_ok and variant in ("auto", "persistent"):
        name, fn = "decode_attention_persistent", lib().bf_decode_attention_persistent
    elif tma_ok and variant != "cp_async":
        name, fn = "decode_attention_tma", lib().bf_decode_attention_tma
    else:
        name, fn = "decode_attention", lib().bf_decode_attention
    if scratch is None:
        max_splits = max(1, -(-int(max_ctx_len) // DECODE_SPLIT_KEYS))
        part_o = torch.empty((n_rows, nh, max_splits, d), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n_rows, nh, max_splits, 2), dtype=torch.float32, device=q.device)
    else:
        part_o, part_ml = scratch
        max_splits = part_o.shape[2]
        _want(part_o, torch.float32, "part_o"); _want(part_ml, torch.float32, "part_ml")
        if (tuple(part_o.shape) != (n_rows, nh, max_splits, d)
                or tuple(part_ml.shape) != (n_rows, nh, max_splits, 2)):
            raise KernelError("decode_attention: scratch must be [n_rows, nh, splits, d] and "
                              "[n_rows, nh, splits, 2]")
    _run(name, fn,
         _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(rows), _ptr(seq_of_token), _ptr(positions),
         _ptr(block_tables), _c_int(block_tables.stride(0)), _ptr(out), _ptr(part_o),
         _ptr(part_ml), _c_int(n_rows), _c_int(nh), _c_int(nkv), _c_int(d),
         _c_int(page_size), _c_int(k_cache.shape[0]), _c_int(window or 0),
         _c_int(max_splits), _c_float(scale), _ptr(err), _stream())
    global _launches
    _launches += 1          # two kernels: the splits and their merge


# scratch for the shares of split prefill attention, per device (grown as needed, up to a limit)
_prefill_split_scratch = {}
_PREFILL_SPLIT_BYTES = 256 << 20


def prefill_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      items: torch.Tensor, n_items: int, max_rows: int,
                      block_tables: torch.Tensor, out: torch.Tensor, nh: int, nkv: int, d: int,
                      window: Optional[int], scale: float, err: torch.Tensor,
                      variant: str = "auto", max_ctx: int = 0, splits: int = 0) -> None:
    """Causal flash attention over the pages for prompt portions (bfloat16 only).
    ``items`` int32 [n, 4]: (request index, first token row, rows, first position).
    ``variant``: ``umma2`` (tcgen05 tensor cores, one CTA per SM with two query tiles sharing a
    K/V ring; head size 128, page sizes 8..64 that divide 64), ``umma`` (two CTAs of one
    query tile per SM; head sizes 64/128, the same page sizes), ``mma_sync`` (every size in
    DECODE_HEAD_DIMS, any page size), or ``auto``: umma2 where it applies and there are
    blocks of 256 rows for most SMs, else umma where it applies, else mma_sync.
    ``max_ctx``: the longest context among the portions, if the caller knows it: few query
    rows after many cached keys then have their keys shared out over several CTAs of the umma2
    kernel, whose partial results a second kernel merges (``splits`` forces a number)."""
    global _launches
    if q.dtype != torch.bfloat16 or d not in DECODE_HEAD_DIMS:
        raise KernelError(f"prefill_attention: bfloat16 and head_dim in {DECODE_HEAD_DIMS} only")
    if variant not in ("auto", "umma2", "umma", "mma_sync"):
        raise KernelError(f"prefill_attention: unknown variant {variant!r}")
    _want(items, torch.int32, "items")
    page_size = k_cache.shape[2]
    umma_ok = (d in (64, 128) and 8 <= page_size <= 64 and 64 % page_size == 0
               and q.is_contiguous() and q.data_ptr() % 16 == 0)
    umma2_ok = umma_ok and d == 128
    if variant == "umma" and not umma_ok or variant == "umma2" and not umma2_ok:
        raise KernelError(f"prefill_attention: the {variant} variant does not take head_dim {d} "
                          f"with pages of {page_size}")
    # umma2 gives an SM one block of 256 rows.  One portion, 32 heads, umma against umma2:
    # 12.8 / 15.0 us at 256 rows from position 0, 20.8 / 20.0 at 512, 44.4 / 29.7 at 1024;
    # after 8192 cached tokens 258 / 162 at 256 rows (58 with the keys shared out, below).
    blocks2 = -(-max_rows // 256) * nh * n_items
    use2 = umma2_ok and (variant == "umma2" or (variant == "auto" and (
        blocks2 >= 120 or max_rows > 256 or max_ctx >= 2048)))
    # Few blocks and long contexts: share the keys of each block out (at least 16 key tiles a
    # share, at most 8 shares, no more CTAs than SMs).
    if splits <= 0:
        splits = 1
        if umma2_ok and variant in ("auto", "umma2") and not window and blocks2 * 2 <= num_sms(q.device):
            splits = max(1, min(8, num_sms(q.device) // blocks2, max_ctx // 1024))
    if splits > 1 and umma2_ok:
        T = q.shape[0]
        need = T * nh * splits
        if need * d * 4 <= _PREFILL_SPLIT_BYTES:
            key = q.device.index
            buf = _prefill_split_scratch.get(key)
            if buf is None or buf[0].numel() < need * d:
                buf = _prefill_split_scratch[key] = (
                    torch.empty(need * d, dtype=torch.float32, device=q.device),
                    torch.empty(need * 2, dtype=torch.float32, device=q.device))
            _run("prefill_attention_umma2", lib().bf_prefill_attention_umma2,
                 _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(items), _c_int(n_items),
                 _c_int(max_rows), _c_int(T), _ptr(block_tables),
                 _c_int(block_tables.stride(0)), _ptr(out), _c_int(nh), _c_int(nkv), _c_int(d),
                 _c_int(page_size), _c_int(k_cache.shape[0]), _c_int(window or 0),
                 _c_float(scale), _c_int(splits), _ptr(buf[0]), _ptr(buf[1]), _ptr(err),
                 _stream())
            _launches += 1          # two kernels: the shares and their merge
            return
    if use2:
        _run("prefill_attention_umma2", lib().bf_prefill_attention_umma2,
             _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(items), _c_int(n_items),
             _c_int(max_rows), _c_int(q.shape[0]), _ptr(block_tables),
             _c_int(block_tables.stride(0)), _ptr(out), _c_int(nh), _c_int(nkv), _c_int(d),
             _c_int(page_size), _c_int(k_cache.shape[0]), _c_int(window or 0), _c_float(scale),
             _c_int(1), None, None, _ptr(err), _stream())
        return
    if umma_ok and variant != "mma_sync":
        name = "prefill_attention_umma"
        _run(name, getattr(lib(), "bf_" + name),
             _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(items), _c_int(n_items),
             _c_int(max_rows), _c_int(q.shape[0]), _ptr(block_tables),
             _c_int(block_tables.stride(0)), _ptr(out), _c_int(nh), _c_int(nkv), _c_int(d),
             _c_int(page_size), _c_int(k_cache.shape[0]), _c_int(window or 0), _c_float(scale),
             _ptr(err), _stream())
        return
    _run("prefill_attention", lib().bf_prefill_attention,
         _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(items), _c_int(n_items), _c_int(max_rows),
         _ptr(block_tables), _c_int(block_tables.stride(0)), _ptr(out), _c_int(nh), _c_int(nkv),
         _c_int(d), _c_int(page_size), _c_int(k_cache.shape[0]), _c_int(window or 0),
         _c_float(scale), _ptr(err), _stream())


# ------------------------------------------------------------- matrix products
def sgemm_nt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T in true 32-bit arithmetic."""
    for t, n in ((a, "a"), (w, "w"), (out, "out")):
        if t.dtype != torch.float32 or t.stride(-1) != 1:
            raise KernelError(f"sgemm_nt: {n} must be float32 with contiguous rows")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"sgemm_nt: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> "
                          f"{tuple(out.shape)} do not agree")
    _run("sgemm_nt", lib().bf_sgemm_nt, _ptr(a), _ptr(w), _ptr(out), _c_int(M), _c_int(N), _c_int(K),
                             _c_ll(a.stride(0)), _c_ll(w.stride(0)), _c_ll(out.stride(0)),
                             _stream())


_num_sms = {}
_err_words = {}


def error_word(device: torch.device) -> torch.Tensor:
    """The device's int32 error word, which kernels OR bits into instead of faulting."""
    w = _err_words.get(device.index)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=device)
        _err_words[device.index] = w
    return w


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, err: torch.Tensor,
              bn: int = 0) -> bool:
    """out[M, N] = x[M, K] @ w[N, K]^T on the tcgen05 tensor cores (bfloat16 in, float
    accumulate, bfloat16 or float32 out).  ``bn``: feature rows per tile (0: chosen by the
    library).  Returns False, having done nothing, for shapes the kernel does not take
    (K not a multiple of 8, misaligned rows)."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_bf16: operands must be bfloat16")
    M, K = x.shape
    N = w.shape[0]
    if (K % 8 or x.stride(1) != 1 or w.stride(1) != 1 or x.stride(0) % 8 or w.stride(0) % 8
            or x.data_ptr() % 16 or w.data_ptr() % 16 or out.stride(1) != 1):
        return False
    sms = _num_sms.get(x.device.index)
    if sms is None:
        sms = torch.cuda.get_device_properties(x.device).multi_processor_count
        _num_sms[x.device.index] = sms
    _run("gemm_bf16_tcgen05", lib().bf_gemm_bf16_tcgen05, _ptr(x), _ptr(w), _ptr(out),
         _c_int(M), _c_int(N), _c_int(K), _c_ll(x.stride(0)), _c_ll(w.stride(0)),
         _c_ll(out.stride(0)), _c_int(_dtype_code(out)), _c_int(bn), _c_int(sms), _ptr(err),
         _stream())
    return True


def gemm_bf16_pair(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, err: torch.Tensor,
                   bn: int = 0, gated: bool = False, accumulate: bool = False) -> bool:
    """out[M, N] = x[M, K] @ w[N, K]^T on pairs of SMs (``tcgen05.mma.cta_group::2``, tiles of
    256 token rows): the product for many token rows.  ``gated``: ``w`` is the stacked
    ``[2 N, K]`` gate/up weight and ``out[M, N] = silu(x w_gate^T) * (x w_up^T)``, bfloat16
    only.  ``accumulate``: ``out`` (float32) ``+=`` the product.  ``bn``: accumulator columns
    per tile (0: chosen by the library).  Returns False, having done nothing, for shapes the
    kernel does not take."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_bf16_pair: operands must be bfloat16")
    if accumulate and (gated or out.dtype != torch.float32):
        raise KernelError("gemm_bf16_pair: accumulate needs a float32 output and no gate")
    M, K = x.shape
    N = out.shape[1]
    if (K % 8 or x.stride(1) != 1 or w.stride(1) != 1 or x.stride(0) % 8 or w.stride(0) % 8
            or x.data_ptr() % 16 or w.data_ptr() % 16 or out.stride(1) != 1
            or out.shape[0] != M or w.shape[0] != (2 * N if gated else N) or w.shape[1] != K
            or (gated and out.dtype != torch.bfloat16)
            or out.dtype not in (torch.bfloat16, torch.float32)):
        return False
    _run("gemm_bf16_pair", lib().bf_gemm_bf16_pair, _ptr(x), _ptr(w), _ptr(out), _c_int(M),
         _c_int(N), _c_int(K), _c_ll(x.stride(0)), _c_ll(w.stride(0)), _c_ll(out.stride(0)),
         _c_int(_dtype_code(out)), _c_int(1 if gated else 0), _c_int(1 if accumulate else 0),
         _c_int(bn), _c_int(num_sms(x.device)), _ptr(err), _stream())
    return True


def gemm_cluster_plan(features: int, K: int, device: torch.device):
    """(bn, cluster) for the split-K cluster product, or None when it does not apply."""
    sms = _num_sms.get(device.index)
    if sms is None:
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        _num_sms[device.index] = sms
    bn, c = _c_int(0), _c_int(0)
    n = lib().bf_gemm_cluster_plan(_c_int(features), _c_int(K), _c_int(sms), ctypes.byref(bn),
                                   ctypes.byref(c))
    return (bn.value, c.value) if n > 0 else None


CLUSTER_MAX_TOKENS = 64


def gemm_bf16_cluster(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, err: torch.Tensor,
                      bn: int, cluster: int) -> bool:
    """out[M, N] = x[M, K] @ w[N, K]^T for M <= 64 with the K range split over clusters of
    ``cluster`` CTAs (partials combined through distributed shared memory).  Returns False,
    having done nothing, for shapes the kernel does not take."""
    M, K = x.shape
    N = w.shape[0]
    if (M > CLUSTER_MAX_TOKENS or K % 8 or x.stride(1) != 1 or w.stride(1) != 1 or x.stride(0) % 8
            or w.stride(0) % 8 or x.data_ptr() % 16 or w.data_ptr() % 16 or out.stride(1) != 1):
        return False
    _run("gemm_bf16_cluster", lib().bf_gemm_bf16_cluster, _ptr(x), _ptr(w), _ptr(out), _c_int(M),
         _c_int(N), _c_int(K), _c_ll(x.stride(0)), _c_ll(w.stride(0)), _c_ll(out.stride(0)),
         _c_int(_dtype_code(out)), _c_int(bn), _c_int(cluster), _ptr(err), _stream())
    return True


def gemm_bf16_cluster_add_norm(x: torch.Tensor, w: torch.Tensor, resid: torch.Tensor,
                               norm_w: torch.Tensor, eps: float, err: torch.Tensor, bn: int,
                               cluster: int):
    """``resid += x @ w^T`` (float32 stream ``[M, N]``), and the next norm's output short of its
    row factor: returns ``(xt, RowScale)`` with ``xt = bfloat16(resid * norm_w)``, or None,
    having done nothing, for shapes the kernel does not take (M <= 64, see
    ``gemm_bf16_cluster``)."""
    M, K = x.shape
    N = w.shape[0]
    if (M > CLUSTER_MAX_TOKENS or K % 8 or x.stride(1) != 1 or w.stride(1) != 1 or x.stride(0) % 8
            or w.stride(0) % 8 or x.data_ptr() % 16 or w.data_ptr() % 16
            or resid.dtype != torch.float32 or resid.shape != (M, N) or resid.stride(1) != 1
            or norm_w.dtype != torch.float32 or norm_w.numel() != N or not norm_w.is_contiguous()):
        return None
    count = -(-N // bn) * cluster
    xt = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    partials = torch.empty((M, count), dtype=torch.float32, device=x.device)
    n = _c_int(0)
    _run("gemm_bf16_cluster_add_norm", lib().bf_gemm_bf16_cluster_add_norm, _ptr(x), _ptr(w),
         _c_int(M), _c_int(N), _c_int(K), _c_ll(x.stride(0)), _c_ll(w.stride(0)), _c_int(bn),
         _c_int(cluster), _ptr(resid), _c_ll(resid.stride(0)), _ptr(norm_w), _ptr(xt),
         _c_ll(xt.stride(0)), _ptr(partials), ctypes.byref(n), _ptr(err), _stream())
    if n.value != count:
        raise KernelError("gemm_bf16_cluster_add_norm: the kernel counts its CTAs differently")
    return xt, RowScale(partials, N, eps)


def num_sms(device: torch.device) -> int:
    sms = _num_sms.get(device.index)
    if sms is None:
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        _num_sms[device.index] = sms
    return sms


def gemm_cluster_qkv_plan(features: int, K: int, d: int, device: torch.device,
                          min_fill: float = 0.6):
    """(bn, cluster, CTAs) for the q/k/v projection with the head norms, the rotation and the
    store into the pages in its epilogue: the narrowest tile of whole heads whose clusters,
    all resident at once, occupy ``min_fill`` of the SMs (or, if none does, the arrangement
    with the most CTAs), or None where the kernel has no such arrangement."""
    bn, c = _c_int(0), _c_int(0)
    sms = num_sms(device)
    n = lib().bf_gemm_cluster_qkv_plan(_c_int(features), _c_int(K), _c_int(d), _c_int(sms),
                                       _c_int(max(1, int(min_fill * sms))), ctypes.byref(bn),
                                       ctypes.byref(c))
    return (bn.value, c.value, n) if n > 0 else None


def gemm_bf16_cluster_qkv(x: torch.Tensor, w: torch.Tensor, q_w: Optional[torch.Tensor],
                          k_w: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor],
                          positions: torch.Tensor, slots: Optional[torch.Tensor],
                          q_out: torch.Tensor, k_cache: Optional[torch.Tensor],
                          v_cache: Optional[torch.Tensor], nh: int, nkv: int, d: int, eps: float,
                          err: torch.Tensor, bn: int, cluster: int,
                          row_scale: Optional[RowScale] = None) -> bool:
    """``qk_norm_rope_kv_write(x @ w^T, ...)`` as one kernel for at most 64 token rows:
    ``w`` is ``[(nh + 2 nkv) d, K]``, or ``[nh d, K]`` with no caches given (queries only).
    Returns False, having done nothing, for what the kernel does not take."""
    M, K = x.shape
    writes = k_cache is not None
    rot_half = 0 if inv_freq is None else inv_freq.numel()
    if (M > CLUSTER_MAX_TOKENS or K % 8 or x.stride(1) != 1 or w.stride(1) != 1 or x.stride(0) % 8
            or w.stride(0) % 8 or x.data_ptr() % 16 or w.data_ptr() % 16 or d % 32 or d > 256
            or rot_half % 32 or 2 * rot_half > d or not q_out.is_contiguous()
            or w.shape[0] != (nh + (2 * nkv if writes else 0)) * d):
        return False
    if writes and not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise KernelError("cache pages must be contiguous")
    page_size = k_cache.shape[2] if writes else 1
    num_slots = k_cache.shape[0] * page_size if writes else 0
    _run("gemm_bf16_cluster_qkv", lib().bf_gemm_bf16_cluster_qkv, _ptr(x), _ptr(w), _c_int(M),
         _c_int(w.shape[0]), _c_int(K), _c_ll(x.stride(0)), _c_ll(w.stride(0)), _c_int(bn),
         _c_int(cluster), _ptr(q_w), _ptr(k_w), _ptr(inv_freq), _c_int(rot_half), _ptr(positions),
         _ptr(slots if writes else None), _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _c_int(nh),
         _c_int(nkv if writes else 0), _c_int(d), _c_int(page_size), _c_ll(num_slots),
         _c_float(eps), *_row_scale_args(row_scale, M), _ptr(err), _stream())
    return True


def gemm_swiglu_plan(inter: int, K: int, device: torch.device):
    """(bn, CTAs) for ``gemm_bf16_swiglu``, or None where its tiles would not fit one wave."""
    bn = _c_int(0)
    n = lib().bf_gemm_swiglu_plan(_c_int(inter), _c_int(K), _c_int(num_sms(device)),
                                  ctypes.byref(bn))
    return (bn.value, n) if n > 0 else None


def gemm_bf16_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor,
                     err: torch.Tensor, bn: int, row_scale: Optional[RowScale] = None) -> bool:
    """``silu_mul(x @ w_gate_up^T)`` as one kernel for at most 64 token rows: ``w_gate_up`` is
    ``[2 I, K]`` with the gate rows first, ``out`` is ``[M, I]``.  Returns False, having done
    nothing, for what the kernel does not take."""
    M, K = x.shape
    I = out.shape[1]
    if (M > CLUSTER_MAX_TOKENS or K % 8 or x.stride(1) != 1 or w_gate_up.stride(1) != 1
            or x.stride(0) % 8 or w_gate_up.stride(0) % 8 or x.data_ptr() % 16
            or w_gate_up.data_ptr() % 16 or out.stride(1) != 1 or out.stride(0) % 8
            or out.data_ptr() % 16 or w_gate_up.shape[0] != 2 * I or out.shape[0] != M
            or out.dtype != torch.bfloat16):
        return False
    _run("gemm_bf16_swiglu", lib().bf_gemm_bf16_swiglu, _ptr(x), _ptr(w_gate_up), _c_int(M),
         _c_int(I), _c_int(K), _c_ll(x.stride(0)), _c_ll(w_gate_up.stride(0)), _c_int(bn),
         _ptr(out), _c_ll(out.stride(0)), *_row_scale_args(row_scale, M), _ptr(err), _stream())
    return True


# -------------------------------------------------------------------- sampling
def repetition_penalty(logits: torch.Tensor, items: torch.Tensor, penalty: torch.Tensor) -> None:
    """items: int32 [n, 3] of (row, token, count)."""
    _want(logits, torch.float32, "logits"); _want(items, torch.int32, "items")
    _run("repetition_penalty", lib().bf_repetition_penalty, _ptr(logits), _c_int(logits.shape[1]), _ptr(items),
                                       _c_int(items.shape[0]), _ptr(penalty), _stream())


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor) -> None:
    _want(logits, torch.float32, "logits"); _want(temperature, torch.float32, "temperature")
    _want(top_k, torch.int32, "top_k"); _want(top_p, torch.float32, "top_p")
    _want(uniform, torch.float32, "uniform"); _want(out, torch.int32, "out")
    R, V = logits.shape
    _run("sample", lib().bf_sample, _ptr(logits), _c_int(R), _c_int(V), _ptr(temperature), _ptr(top_k),
                           _ptr(top_p), _ptr(uniform), _ptr(out), _stream())
