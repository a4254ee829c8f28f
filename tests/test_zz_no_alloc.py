"""The decode-attention entry point that allocates nothing, called through its C symbol.

Some users of the library cannot allocate device memory when they call it: their
own pool took the whole GPU at start-up, or they sit in a loop that must not pay
cudaMalloc's device-wide synchronisation, or they come from a host language that
can only pass pointers it already owns.  For them ``bf_decode_attention_static``
keeps the scratch for the key splits in an 8 MiB array inside the library.

This file is collected last on purpose: the array keeps what earlier calls left
in it, so the test has to pass after everything else has run as well as alone in
a fresh process.  It checks two calls in a row (different shapes, so the second
one finds the first one's leftovers) against the ordinary entry point, which gets
its scratch from the caller.
"""
import ctypes

import pytest
import torch

from test_kernels_gpu import BF16, _attention_case, _close

pytestmark = pytest.mark.gpu

SCRATCH_BYTES = 8 << 20


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _call_static(lib, q, kc, vc, rows, n_rows, sot, pos, bt, out, nh, nkv, d, window, max_splits,
                 err):
    fn = lib.bf_decode_attention_static
    fn.restype = ctypes.c_int
    return fn(_p(q), _p(kc), _p(vc), _p(rows), _p(sot), _p(pos), _p(bt),
              ctypes.c_int(bt.stride(0)), _p(out), ctypes.c_int(n_rows), ctypes.c_int(nh),
              ctypes.c_int(nkv), ctypes.c_int(d), ctypes.c_int(kc.shape[2]),
              ctypes.c_int(kc.shape[0]), ctypes.c_int(window or 0), ctypes.c_int(max_splits),
              ctypes.c_float(d ** -0.5), _p(err),
              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def _message(lib, code):
    fn = lib.bf_decode_attention_static_error
    fn.restype = ctypes.c_char_p
    return fn(ctypes.c_int(code)).decode()


def test_static_scratch_entry_point_matches_the_ordinary_one(cuda_device):
    from binfer_b200.csrc import ops
    lib = ops.lib()
    cases = [
        # nh, nkv, d, page, window, contexts
        (8, 2, 128, 16, None, [1, 127, 128, 129, 300, 1000]),
        (6, 1, 64, 8, 200, [513, 45, 260]),       # other shape: finds the first call's leftovers
    ]
    for nh, nkv, d, ps, window, ctxs in cases:
        q, kc, vc, sot, pos, bt, ref = _attention_case(
            cuda_device, BF16, nh, nkv, d, ps, ctxs, [1] * len(ctxs), window, spike=True, seed=9)
        err = torch.zeros(1, dtype=torch.int32, device=cuda_device)
        max_splits = -(-max(ctxs) // 128)
        want = torch.zeros_like(q)
        ops.decode_attention(q, kc, vc, None, len(ctxs), sot, pos, bt, want, nh, nkv, d, window,
                             d ** -0.5, max(ctxs), err, variant="cp_async")
        got = torch.zeros_like(q)
        code = _call_static(lib, q, kc, vc, None, len(ctxs), sot, pos, bt, got, nh, nkv, d,
                            window, max_splits, err)
        assert code == 0, _message(lib, code)
        torch.cuda.synchronize()
        assert int(err.item()) == 0
        _close(got, want.double().cpu(), BF16)     # against the existing entry point
        _close(got, ref, BF16)                     # and against the plain reference
        # a subset of the rows, named by index: those rows get the same bits, the others nothing
        rows = torch.tensor([2, 0], dtype=torch.int32, device=cuda_device)
        some = torch.zeros_like(q)
        code = _call_static(lib, q, kc, vc, rows, 2, sot, pos, bt, some, nh, nkv, d, window,
                            max_splits, err)
        assert code == 0, _message(lib, code)
        torch.cuda.synchronize()
        assert torch.equal(some[2], got[2]) and torch.equal(some[0], got[0])
        assert float(some[1].abs().max()) == 0.0


def test_static_scratch_entry_point_flags_too_few_splits(cuda_device):
    """max_splits is the caller's word; a row whose keys need more than it says sets the
    error word's bit 16 and loses its far keys, instead of reading or writing past the
    room the call was sized for."""
    from binfer_b200.csrc import ops
    lib = ops.lib()
    nh, nkv, d, ps = 8, 2, 128, 16
    q, kc, vc, sot, pos, bt, ref = _attention_case(cuda_device, BF16, nh, nkv, d, ps, [200, 90],
                                                   [1, 1], None, seed=2)
    err = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    out = torch.zeros_like(q)
    code = _call_static(lib, q, kc, vc, None, 2, sot, pos, bt, out, nh, nkv, d, None, 1, err)
    assert code == 0, _message(lib, code)
    torch.cuda.synchronize()
    assert int(err.item()) == 16
    _close(out[1], ref[1], BF16)


def test_static_scratch_entry_point_refuses_what_does_not_fit(cuda_device):
    from binfer_b200.csrc import ops
    lib = ops.lib()
    nh, nkv, d, ps = 32, 8, 128, 16
    q, kc, vc, sot, pos, bt, _ = _attention_case(cuda_device, BF16, nh, nkv, d, ps, [40, 50],
                                                 [1, 1], None, seed=1)
    err = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    out = torch.full_like(q, 7.0)
    too_many_splits = SCRATCH_BYTES // (2 * nh * (d + 2) * 4) + 1
    code = _call_static(lib, q, kc, vc, None, 2, sot, pos, bt, out, nh, nkv, d, None,
                        too_many_splits, err)
    assert code == -1 and "8 MiB" in _message(lib, code)
    torch.cuda.synchronize()
    assert bool((out == 7.0).all()), "a refused call must not launch anything"
    assert _call_static(lib, q, kc, vc, None, 2, sot, pos, bt, out, nh, nkv, 48, None, 1,
                        err) == -2
    # the largest call that fits still runs
    code = _call_static(lib, q, kc, vc, None, 2, sot, pos, bt, out, nh, nkv, d, None,
                        too_many_splits - 1, err)
    assert code == 0, _message(lib, code)
    torch.cuda.synchronize()
