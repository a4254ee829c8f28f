"""Each CUDA kernel alone against a plain float64 reference, at sizes other than the engine's."""
import math

import pytest
import torch

import qwen3_plain as P

pytestmark = pytest.mark.gpu

BF16, F32 = torch.bfloat16, torch.float32
TOL = {F32: 2e-6, BF16: 1.2e-2}     # relative to the largest reference magnitude


def _close(got, ref, dtype, scale=1.0):
    err = float((got.double().cpu() - ref.double().cpu()).abs().max())
    mag = float(ref.double().abs().max()) or 1.0
    assert err <= TOL[dtype] * scale * mag, f"error {err:.3g} vs magnitude {mag:.3g}"


def _err(dev):
    return torch.zeros(1, dtype=torch.int32, device=dev)


# ------------------------------------------------------------------ elementwise
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_embed_gather(cuda_device, dtype):
    from binfer_b200.csrc import ops
    table = torch.randn(301, 100, device=cuda_device).to(dtype)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32, device=cuda_device)
    out = torch.empty(5, 100, device=cuda_device)
    err = _err(cuda_device)
    ops.embed_gather(table, ids, out, 1.0, err)
    assert torch.equal(out, table.float()[ids.long()])
    assert int(err.item()) == 0
    bad = torch.tensor([3, 301], dtype=torch.int32, device=cuda_device)
    out2 = torch.ones(2, 100, device=cuda_device)
    ops.embed_gather(table, bad, out2, 1.0, err)
    assert int(err.item()) == 1 and float(out2[1].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("H", [100, 1536, 5000])
def test_add_rmsnorm(cuda_device, dtype, H):
    from binfer_b200.csrc import ops
    resid = torch.randn(9, H, device=cuda_device)
    delta = torch.randn(9, H, device=cuda_device).to(dtype)
    w = 1 + 0.1 * torch.randn(H, device=cuda_device)
    r0 = resid.clone()
    out = torch.empty(9, H, device=cuda_device, dtype=dtype)
    ops.add_rmsnorm(resid, delta, w, out, 1e-5)
    x = r0.double() + delta.double()
    _close(resid, x, F32)
    _close(out, P.rms_norm(x, w.double(), 1e-5), dtype)
    # selected rows, no pending add, stream untouched
    rows = torch.tensor([8, 2], dtype=torch.int32, device=cuda_device)
    keep = resid.clone()
    out2 = torch.empty(2, H, device=cuda_device, dtype=dtype)
    ops.add_rmsnorm(resid, None, w, out2, 1e-6, rows=rows, write_back=False)
    assert torch.equal(resid, keep)
    _close(out2, P.rms_norm(keep.double()[[8, 2]], w.double(), 1e-6), dtype)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_silu_mul_and_residual_add(cuda_device, dtype):
    from binfer_b200.csrc import ops
    gu = (3 * torch.randn(7, 2 * 150, device=cuda_device)).to(dtype)
    out = torch.empty(7, 150, device=cuda_device, dtype=dtype)
    ops.silu_mul(gu, out)
    g, u = gu.double()[:, :150], gu.double()[:, 150:]
    _close(out, g / (1 + torch.exp(-g)) * u, dtype)
    resid = torch.randn(7, 150, device=cuda_device)
    want = resid.double() + out.double()
    ops.residual_add(resid, out)
    _close(resid, want, F32)


@pytest.mark.parametrize("M", [1, 7, 16, 63, 65, 130])
def test_sgemm_true_float32(cuda_device, M):
    from binfer_b200.csrc import ops
    N, K = 300, 203
    a = torch.randn(130, K, device=cuda_device)
    w = torch.randn(N, K, device=cuda_device)
    out = torch.empty(M, N, device=cuda_device)
    ops.sgemm_nt(a[:M], w, out)
    ref = a[:M].double() @ w.double().T
    assert float((out.double() - ref).abs().max()) <= 2e-6 * float(ref.abs().max()) * math.sqrt(K)
    # a row's result does not depend on how many rows share the call (one order of summation)
    big = torch.empty(130, N, device=cuda_device)
    ops.sgemm_nt(a, w, big)
    assert torch.equal(out, big[:M])


# ------------------------------------------------------- q/k norm, rotation, cache write
@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("nh,nkv,d,rot,norm", [(3, 1, 16, 16, True), (4, 2, 48, 24, True),
                                               (2, 2, 128, 128, False), (5, 5, 80, 0, True),
                                               (8, 2, 128, 128, True), (3, 1, 128, 64, True)])
def test_qk_norm_rope_kv_write(cuda_device, dtype, nh, nkv, d, rot, norm):
    from binfer_b200.csrc import ops
    T, ps, pages, eps, theta = 11, 4, 9, 1e-5, 5000.0
    dev = cuda_device
    qkv = torch.randn(T, (nh + 2 * nkv) * d, device=dev).to(dtype)
    qw = (1 + 0.1 * torch.randn(d, device=dev)) if norm else None
    kw = (1 + 0.1 * torch.randn(d, device=dev)) if norm else None
    pos = torch.tensor([0, 1, 2, 3, 40, 41, 1000, 7, 8, 9, 10], dtype=torch.int32, device=dev)
    slots = torch.randperm(pages * ps)[:T].to(torch.int32).to(dev)
    slots[3] = -1                                   # this token is not written
    inv = None
    if rot:
        i = torch.arange(rot // 2, dtype=torch.float64)
        inv = (theta ** (-2.0 * i / rot)).float().to(dev)
    kc = torch.zeros(pages, nkv, ps, d, device=dev, dtype=dtype)
    vc = torch.zeros_like(kc)
    q_out = torch.empty(T, nh * d, device=dev, dtype=dtype)
    err = _err(dev)
    ops.qk_norm_rope_kv_write(qkv, qw, kw, inv, pos, slots, q_out, kc, vc, nh, nkv, d, eps, err)
    assert int(err.item()) == 0
    x = qkv.double().cpu()
    q = x[:, :nh * d].view(T, nh, d)
    k = x[:, nh * d:(nh + nkv) * d].view(T, nkv, d)
    v = x[:, (nh + nkv) * d:].view(T, nkv, d)
    if norm:
        q, k = P.rms_norm(q, qw.double().cpu(), eps), P.rms_norm(k, kw.double().cpu(), eps)
    if rot:
        ang = P.rope_angles(pos.cpu(), rot, theta)
        q, k = P.apply_rope(q, ang), P.apply_rope(k, ang)
    _close(q_out.view(T, nh, d), q, dtype)
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        _close(kc[s // ps, :, s % ps], k[t], dtype)
        _close(vc[s // ps, :, s % ps], v[t], dtype)
    assert float(kc.abs().sum(dim=(1, 3)).flatten().count_nonzero()) == T - 1


@pytest.mark.parametrize("nh,nkv,norm", [(8, 2, True), (32, 8, True), (5, 1, True), (64, 8, True),
                                         (3, 3, False)])
def test_qk_norm_rope_kv_write_many_tokens(cuda_device, nh, nkv, norm):
    """Heads of 128 and more than 64 tokens: a block per token whose warps walk the heads, six
    of them asked for at a time.  Odd head counts, 80 heads; some tokens are not written;
    positions are far apart."""
    from binfer_b200.csrc import ops
    T, d, ps, eps, theta = 203, 128, 16, 1e-6, 1e6
    dev = cuda_device
    g = torch.Generator().manual_seed(nh)
    qkv = torch.randn(T, (nh + 2 * nkv) * d, generator=g).to(BF16).to(dev)
    qw = (1 + 0.1 * torch.randn(d, generator=g)).to(dev) if norm else None
    kw = (1 + 0.1 * torch.randn(d, generator=g)).to(dev) if norm else None
    pos = (torch.arange(T) * 37 % 5000).to(torch.int32).to(dev)
    pages = T // ps + 3
    slots = torch.randperm(pages * ps, generator=g)[:T].to(torch.int32)
    slots[7] = slots[100] = -1
    slots = slots.to(dev)
    i = torch.arange(d // 2, dtype=torch.float64)
    inv = (theta ** (-2.0 * i / d)).float().to(dev)
    kc = torch.zeros(pages, nkv, ps, d, device=dev, dtype=BF16)
    vc = torch.zeros_like(kc)
    q_out = torch.empty(T, nh * d, device=dev, dtype=BF16)
    err = _err(dev)
    ops.qk_norm_rope_kv_write(qkv, qw, kw, inv, pos, slots, q_out, kc, vc, nh, nkv, d, eps, err)
    assert int(err.item()) == 0
    x = qkv.double().cpu()
    q = x[:, :nh * d].view(T, nh, d)
    k = x[:, nh * d:(nh + nkv) * d].view(T, nkv, d)
    v = x[:, (nh + nkv) * d:].view(T, nkv, d)
    if norm:
        q, k = P.rms_norm(q, qw.double().cpu(), eps), P.rms_norm(k, kw.double().cpu(), eps)
    ang = P.rope_angles(pos.cpu(), d, theta)
    q, k = P.apply_rope(q, ang), P.apply_rope(k, ang)
    _close(q_out.view(T, nh, d), q, BF16)
    sl = slots.cpu()
    live = sl >= 0
    got_k = kc.cpu()[sl[live] // ps, :, sl[live] % ps]
    got_v = vc.cpu()[sl[live] // ps, :, sl[live] % ps]
    _close(got_k, k[live], BF16)
    _close(got_v, v[live], BF16)
    assert int(kc.abs().sum(dim=(1, 3)).flatten().count_nonzero()) == int(live.sum())


# ----------------------------------------------------------------------- attention
def _paged(k, v, ps, dev, dtype, seed=0, neighbours=False):
    """Scatter dense k, v ``[n, nkv, d]`` of one request into shuffled pages (or, with
    ``neighbours``, into pages that lie side by side in the pool).
    Returns caches ``[pages, nkv, ps, d]`` and the block table."""
    n, nkv, d = k.shape
    n_pages = -(-n // ps)
    total = n_pages + 5
    g = torch.Generator().manual_seed(seed)
    ids = (torch.randperm(total - 1, generator=g)[:n_pages] + 1).tolist()   # page 0 unused
    if neighbours:
        ids = list(range(3, 3 + n_pages))
    kc = torch.randn(total, nkv, ps, d, generator=g).to(dtype)              # junk elsewhere
    vc = torch.randn(total, nkv, ps, d, generator=g).to(dtype)
    for j in range(n):
        kc[ids[j // ps], :, j % ps] = k[j].to(dtype)
        vc[ids[j // ps], :, j % ps] = v[j].to(dtype)
    return kc.to(dev), vc.to(dev), ids


def _attention_case(dev, dtype, nh, nkv, d, ps, ctxs, qlens, window, spike=False, seed=0,
                    neighbours=False):
    """Requests with contexts ``ctxs``, the last ``qlens`` tokens of each being queries."""
    g = torch.Generator().manual_seed(seed)
    ks, vs, qs, tables, refs = [], [], [], [], []
    kcs, vcs = [], []
    page_base = 0
    for b, (n, ql) in enumerate(zip(ctxs, qlens)):
        k = torch.randn(n, nkv, d, generator=g).to(dtype).double()
        v = torch.randn(n, nkv, d, generator=g).to(dtype).double()
        q = torch.randn(n, nh, d, generator=g).to(dtype).double()
        if spike and n > 40:
            # one far key stands out: its score beats hundreds of others.  With a window it
            # is the first key inside the last query's window, and the key just outside
            # stands out even more, so reading one key too many shows as well.
            far = 3 if window is None else max(0, n - window)
            k[far] = 0
            k[far, :, 0] = 32.0
            q[-1, :, 0] = 16.0
            v[far] = 5.0
            if window is not None and far > 0:
                k[far - 1] = 0
                k[far - 1, :, 0] = 64.0
                v[far - 1] = -7.0
        ref = P.causal_attention(q, k, v, d ** -0.5, window)[n - ql:]
        kc, vc, ids = _paged(k, v, ps, "cpu", dtype, seed + b, neighbours)
        kcs.append(kc)
        vcs.append(vc)
        tables.append([i + page_base for i in ids])
        page_base += kc.shape[0]
        qs.append(q[n - ql:])
        refs.append(ref)
    width = max(len(t) for t in tables)
    bt = torch.zeros(len(ctxs), width, dtype=torch.int32)
    for b, t in enumerate(tables):
        bt[b, :len(t)] = torch.tensor(t, dtype=torch.int32)
    q_all = torch.cat(qs).to(dtype).reshape(-1, nh * d).to(dev)
    pos = torch.cat([torch.arange(n - ql, n) for n, ql in zip(ctxs, qlens)]).to(torch.int32).to(dev)
    sot = torch.cat([torch.full((ql,), b) for b, ql in enumerate(qlens)]).to(torch.int32).to(dev)
    return (q_all, torch.cat(kcs).to(dev), torch.cat(vcs).to(dev), sot, pos, bt.to(dev),
            torch.cat(refs).reshape(-1, nh * d))


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("nh,nkv,d,ps,window,spike", [
    (4, 2, 16, 16, None, False), (6, 1, 32, 8, None, True), (5, 5, 48, 4, 24, True),
    (8, 2, 128, 16, None, True), (3, 3, 80, 5, 33, False), (2, 1, 256, 16, 100, True)])
def test_paged_attention_generic(cuda_device, dtype, nh, nkv, d, ps, window, spike):
    from binfer_b200.csrc import ops
    ctxs, qlens = [70, 1, 129, 300], [70, 1, 5, 2]
    q, kc, vc, sot, pos, bt, ref = _attention_case(cuda_device, dtype, nh, nkv, d, ps, ctxs,
                                                   qlens, window, spike)
    out = torch.empty_like(q)
    err = _err(cuda_device)
    ops.paged_attention_generic(q, kc, vc, sot, pos, bt, out, nh, nkv, d, window, d ** -0.5, err)
    assert int(err.item()) == 0
    _close(out, ref, dtype)


@pytest.mark.parametrize("nh,nkv,d,ps,window,spike", [
    (4, 2, 32, 16, None, False), (6, 1, 32, 8, None, True), (8, 2, 128, 16, None, True),
    (32, 8, 128, 16, None, False), (5, 5, 96, 4, 24, True), (3, 3, 64, 5, 200, True),
    (2, 1, 256, 16, 100, True), (20, 1, 64, 16, None, True), (4, 4, 128, 64, 130, True)])
@pytest.mark.parametrize("variant", ["cp_async", "tma", "persistent"])
def test_decode_attention_split_kv(cuda_device, nh, nkv, d, ps, window, spike, variant):
    """Contexts on both sides of the 128-key split edge, and long ones; every way of
    fetching the tiles."""
    from binfer_b200.csrc import ops
    if variant != "cp_async" and not (d in (64, 128, 256) and ps >= 8 and 128 % ps == 0):
        pytest.skip(f"the {variant} variant does not take this head or page size")
    if variant == "persistent" and nh // nkv > 16:
        pytest.skip("the persistent variant takes at most 16 heads per kv head")
    ctxs = [1, 127, 128, 129, 300, 1000, 45]
    qlens = [1] * len(ctxs)
    q, kc, vc, sot, pos, bt, ref = _attention_case(cuda_device, BF16, nh, nkv, d, ps, ctxs,
                                                   qlens, window, spike, seed=3)
    out = torch.zeros_like(q)
    err = _err(cuda_device)
    ops.decode_attention(q, kc, vc, None, len(ctxs), sot, pos, bt, out, nh, nkv, d, window,
                         d ** -0.5, max(ctxs) + 500, err, variant=variant)
    assert int(err.item()) == 0
    _close(out, ref, BF16)
    # a subset of rows, given by index, gives the same bits for those rows
    rows = torch.tensor([5, 2, 4], dtype=torch.int32, device=cuda_device)
    out2 = torch.zeros_like(q)
    ops.decode_attention(q, kc, vc, rows, 3, sot, pos, bt, out2, nh, nkv, d, window,
                         d ** -0.5, max(ctxs), err, variant=variant)
    for r in (5, 2, 4):
        assert torch.equal(out2[r], out[r])
    assert float(out2[0].abs().max()) == 0.0


@pytest.mark.parametrize("nh,nkv,d,ps,window", [
    (8, 2, 128, 16, None), (32, 8, 128, 16, 300), (6, 3, 64, 8, None), (4, 4, 256, 32, None),
    (8, 4, 128, 64, 1000)])
def test_decode_attention_with_pages_side_by_side(cuda_device, nh, nkv, d, ps, window):
    """Tiles whose pages are neighbours in the pool arrive as one box: the same bits as with
    the pages scattered (one box a page), and the plain result.  Contexts that end inside a
    tile, rows shorter than a tile, a window that starts inside one."""
    from binfer_b200.csrc import ops
    ctxs = [1, 127, 128, 129, 300, 1000, 45, 2050, 640]
    qlens = [1] * len(ctxs)
    outs = []
    for neighbours in (True, False):
        q, kc, vc, sot, pos, bt, ref = _attention_case(
            cuda_device, BF16, nh, nkv, d, ps, ctxs, qlens, window, True, seed=13,
            neighbours=neighbours)
        out = torch.zeros_like(q)
        err = _err(cuda_device)
        ops.decode_attention(q, kc, vc, None, len(ctxs), sot, pos, bt, out, nh, nkv, d, window,
                             d ** -0.5, max(ctxs), err, variant="persistent")
        assert int(err.item()) == 0
        _close(out, ref, BF16)
        outs.append(out)
    assert torch.equal(outs[0], outs[1]), "the result depends on where the pages lie"


@pytest.mark.parametrize("nh,nkv,d,ps,window", [
    (8, 4, 128, 16, None), (12, 4, 64, 32, 700), (4, 2, 256, 8, None), (16, 1, 128, 128, None)])
def test_decode_attention_persistent_ring_wraps(cuda_device, nh, nkv, d, ps, window):
    """So many (row, kv head, split) items that every resident CTA takes more of them than its
    ring of tile slots holds, with rows of very different lengths; compared with the plain
    result and, bit for bit, with the one-CTA-per-split kernel's partial sums merged the
    same way."""
    from binfer_b200.csrc import ops
    ctxs = [2900, 1, 1500, 130, 3001, 777, 2048, 64, 2500, 3, 1999, 2300] * 2
    qlens = [1] * len(ctxs)
    q, kc, vc, sot, pos, bt, ref = _attention_case(cuda_device, BF16, nh, nkv, d, ps, ctxs,
                                                   qlens, window, True, seed=11)
    err = _err(cuda_device)
    out = torch.zeros_like(q)
    ops.decode_attention(q, kc, vc, None, len(ctxs), sot, pos, bt, out, nh, nkv, d, window,
                         d ** -0.5, max(ctxs), err, variant="persistent")
    assert int(err.item()) == 0
    _close(out, ref, BF16)
    again = torch.zeros_like(q)
    ops.decode_attention(q, kc, vc, None, len(ctxs), sot, pos, bt, again, nh, nkv, d, window,
                         d ** -0.5, max(ctxs), err, variant="persistent")
    assert torch.equal(out, again), "the result depends on timing"


@pytest.mark.parametrize("window", [None, 5000])
@pytest.mark.parametrize("variant", ["cp_async", "tma", "persistent"])
def test_decode_attention_more_splits_than_one_merge_pass(cuda_device, variant, window):
    """Contexts beyond 16384 keys: the merge kernel's shape for many splits, more of them than
    a lane asks for at once, and (with a window) a first split that is not split 0.  One key
    far back is made to stand out, so a lost pass would show."""
    from binfer_b200.csrc import ops
    nh, nkv, d, ps = 4, 2, 64, 64
    ctxs, qlens = [20000, 16385, 300], [1, 1, 1]
    q, kc, vc, sot, pos, bt, ref = _attention_case(cuda_device, BF16, nh, nkv, d, ps, ctxs,
                                                   qlens, window, True, seed=5)
    out = torch.zeros_like(q)
    err = _err(cuda_device)
    ops.decode_attention(q, kc, vc, None, len(ctxs), sot, pos, bt, out, nh, nkv, d, window,
                         d ** -0.5, max(ctxs), err, variant=variant)
    assert int(err.item()) == 0
    _close(out, ref, BF16)


@pytest.mark.parametrize("variant", ["cp_async", "tma", "persistent"])
def test_decode_attention_flags_a_row_beyond_its_scratch(cuda_device, variant):
    """Scratch with room for one split and a row of 200 keys, which needs two: the error
    word's bit says so, nothing behind the scratch is touched, and the row that fits is
    right all the same."""
    from binfer_b200.csrc import ops
    nh, nkv, d, ps = 8, 2, 128, 16
    ctxs = [200, 90]
    q, kc, vc, sot, pos, bt, ref = _attention_case(cuda_device, BF16, nh, nkv, d, ps, ctxs,
                                                   [1, 1], None, seed=21)
    cells = len(ctxs) * nh * 1
    buf = torch.full((cells * (d + 2) + 8192,), 777.0, dtype=torch.float32, device=cuda_device)
    part_o = buf[:cells * d].view(len(ctxs), nh, 1, d)
    part_ml = buf[cells * d:cells * (d + 2)].view(len(ctxs), nh, 1, 2)
    out = torch.zeros_like(q)
    err = _err(cuda_device)
    ops.decode_attention(q, kc, vc, None, len(ctxs), sot, pos, bt, out, nh, nkv, d, None,
                         d ** -0.5, max(ctxs), err, variant=variant, scratch=(part_o, part_ml))
    torch.cuda.synchronize()
    assert int(err.item()) == 16
    err.zero_()
    assert bool((buf[cells * (d + 2):] == 777.0).all()), "memory behind the scratch was written"
    _close(out[1], ref[1], BF16)
    assert bool(torch.isfinite(out.float()).all())


@pytest.mark.parametrize("M,N,K,bn,c", [(8, 4096, 4096, 128, 4), (3, 200, 512, 64, 2),
                                        (16, 1000, 320, 80, 1), (64, 4096, 4096, 128, 4),
                                        (37, 1024, 2048, 64, 4), (27, 520, 1024, 64, 2),
                                        (32, 4096, 4096, 128, 4)])
def test_gemm_cluster_adds_into_the_stream_and_prepares_the_norm(cuda_device, M, N, K, bn, c):
    """resid += x w^T in float; xt = bf16(resid * norm_w); the partial sums of squares add up
    to the rows' sums, so that xt times the factor is the RMSNorm of the new stream."""
    from binfer_b200.csrc import ops
    g = torch.Generator().manual_seed(N + K)
    x = torch.randn(M, K, generator=g).to(BF16).to(cuda_device)
    w = (0.05 * torch.randn(N, K, generator=g)).to(BF16).to(cuda_device)
    resid0 = (3.0 * torch.randn(M, N, generator=g)).to(cuda_device)
    nw = (1.0 + 0.1 * torch.randn(N, generator=g)).to(cuda_device)
    eps = 1e-5
    resid = resid0.clone()
    err = ops.error_word(cuda_device)
    got = ops.gemm_bf16_cluster_add_norm(x, w, resid, nw, eps, err, bn, c)
    assert got is not None and int(err.item()) == 0
    xt, scale = got
    want = resid0.double().cpu() + x.double().cpu() @ w.double().cpu().T
    assert float((resid.double().cpu() - want).abs().max()) <= 4e-7 * math.sqrt(K) * float(want.abs().max())
    assert scale.partials.shape == (M, -(-N // bn) * c) and scale.width == N
    ss = scale.partials.double().sum(1).cpu()
    assert torch.allclose(ss, (want ** 2).sum(1), rtol=1e-5)
    normed = want * torch.rsqrt((want ** 2).mean(1, keepdim=True) + eps) * nw.double().cpu()
    _close(xt.float() * scale.factors().unsqueeze(1), normed, BF16)
    # the factor applied by the kernels that come after the next product
    I = 264
    gu = torch.randn(M, 2 * I, generator=g).to(BF16).to(cuda_device)
    out = torch.empty(M, I, device=cuda_device, dtype=BF16)
    ops.silu_mul(gu, out, row_scale=scale)
    f = scale.factors().double().cpu().unsqueeze(1)
    gd = gu.double().cpu() * f
    _close(out, gd[:, :I] / (1 + torch.exp(-gd[:, :I])) * gd[:, I:], BF16)


@pytest.mark.parametrize("T,nh,nkv,d,rot,K,bn,c,norm,scaled", [
    (8, 32, 8, 128, 128, 4096, 128, 2, True, True),      # the 8B decode step's arrangement
    (5, 6, 2, 64, 64, 1024, 128, 2, True, False),        # two heads a tile
    (13, 5, 1, 96, 64, 1280, 192, 4, True, True),        # a rotation over part of the head
    (16, 3, 3, 256, 256, 512, 256, 1, False, False),     # one CTA a tile, no head norms
    (37, 7, 1, 128, 0, 2304, 128, 5, True, True),        # token rows beyond 32, no rotation
    (21, 4, 2, 64, 64, 1024, 128, 2, True, True),        # 17 to 32 token rows
    (2, 4, 0, 128, 128, 640, 256, 2, True, False),       # queries only: another layer's pages
    (1, 8, 2, 32, 0, 768, 32, 3, False, True),           # fewer tokens than CTAs in a cluster
])
def test_gemm_cluster_qkv_norms_turns_and_stores(cuda_device, T, nh, nkv, d, rot, K, bn, c, norm,
                                                 scaled):
    """The q/k/v projection with its epilogue against the product followed by the plain
    head norm, rotation and store: q, and every page slot of k and v (untouched slots
    stay zero, a token with a negative slot is not stored)."""
    from binfer_b200.csrc import ops
    dev, ps, eps, theta = cuda_device, 4, 1e-5, 5000.0
    pages = -(-T // ps) + 3
    g = torch.Generator().manual_seed(T * 1000 + K)
    x = torch.randn(T, K, generator=g).to(BF16).to(dev)
    w = (torch.randn((nh + 2 * nkv) * d, K, generator=g) / math.sqrt(K)).to(BF16).to(dev)
    qw = (1 + 0.1 * torch.randn(d, generator=g)).to(dev) if norm else None
    kw = (1 + 0.1 * torch.randn(d, generator=g)).to(dev) if norm else None
    pos = torch.randint(0, 3000, (T,), generator=g).to(torch.int32).to(dev)
    slots = torch.randperm(pages * ps, generator=g)[:T].to(torch.int32).to(dev)
    if T > 3:
        slots[3] = -1
    inv = None
    if rot:
        i = torch.arange(rot // 2, dtype=torch.float64)
        inv = (theta ** (-2.0 * i / rot)).float().to(dev)
    scale = None
    factor = torch.ones(T, dtype=torch.float64)
    if scaled:
        partials = (torch.rand(T, 37, generator=g) * 40).to(dev)
        scale = ops.RowScale(partials, 1536, 1e-6)
        factor = scale.factors().double().cpu()
    kc = torch.zeros(pages, max(nkv, 1), ps, d, device=dev, dtype=BF16) if nkv else None
    vc = torch.zeros_like(kc) if nkv else None
    q_out = torch.empty(T, nh * d, device=dev, dtype=BF16)
    err = _err(dev)
    assert ops.gemm_bf16_cluster_qkv(x, w, qw, kw, inv, pos, slots if nkv else None, q_out, kc, vc,
                                     nh, nkv, d, eps, err, bn, c, row_scale=scale)
    assert int(err.item()) == 0
    y = (x.double().cpu() @ w.double().cpu().T) * factor[:, None]
    q = y[:, :nh * d].view(T, nh, d)
    k = y[:, nh * d:(nh + nkv) * d].view(T, nkv, d)
    v = y[:, (nh + nkv) * d:].view(T, nkv, d)
    if norm:
        q = P.rms_norm(q, qw.double().cpu(), eps)
        k = P.rms_norm(k, kw.double().cpu(), eps) if nkv else k
    if rot:
        ang = P.rope_angles(pos.cpu(), rot, theta)
        q = P.apply_rope(q, ang)
        k = P.apply_rope(k, ang) if nkv else k
    _close(q_out.view(T, nh, d), q, BF16)
    if not nkv:
        return
    stored = 0
    for t in range(T):
        s_ = int(slots[t])
        if s_ < 0:
            continue
        stored += 1
        _close(kc[s_ // ps, :, s_ % ps], k[t], BF16)
        _close(vc[s_ // ps, :, s_ % ps], v[t], BF16)
    assert int(kc.abs().sum(dim=(1, 3)).flatten().count_nonzero()) == stored
    assert int(vc.abs().sum(dim=(1, 3)).flatten().count_nonzero()) == stored


def test_gemm_cluster_qkv_plan_keeps_whole_heads(cuda_device):
    from binfer_b200.csrc import ops
    sms = ops.num_sms(cuda_device)
    for features, K, d in [(6144, 4096, 128), (2560, 1536, 128), (10240, 5120, 128),
                           (1536, 1024, 64), (1280, 2048, 256), (480, 640, 96)]:
        plan = ops.gemm_cluster_qkv_plan(features, K, d, cuda_device)
        assert plan is not None, (features, K, d)
        bn, c, ctas = plan
        assert bn % d == 0 and bn <= 256 and 1 <= c <= 8 and (K // 64) // c >= 4
        assert ctas == -(-features // bn) * c <= sms
    assert ops.gemm_cluster_qkv_plan(4096, 4096, 80, cuda_device) is None     # not whole warps


@pytest.mark.parametrize("T,I,K,bn,scaled", [
    (8, 12288, 4096, 0, True),        # the 8B decode step's shape, the plan's tile
    (5, 1000, 512, 0, False),         # outputs that are no multiple of the tile
    (16, 2504, 320, 48, True),        # 24 outputs a tile: the last chunk of a tile is cut
    (37, 264, 1024, 256, True),       # token rows beyond 32; one tile holds part of the outputs
    (29, 1000, 512, 0, True),         # 17 to 32 token rows: 64-row products, two lane quarters
    (1, 4480, 1536, 112, False),
])
def test_gemm_swiglu_matches_product_then_activation(cuda_device, T, I, K, bn, scaled):
    """silu(f g) * (f u) of the stacked gate/up product, straight from tensor memory."""
    from binfer_b200.csrc import ops
    dev = cuda_device
    g = torch.Generator().manual_seed(I + K + T)
    x = torch.randn(T, K, generator=g).to(BF16).to(dev)
    w = (2.0 * torch.randn(2 * I, K, generator=g) / math.sqrt(K)).to(BF16).to(dev)
    scale, f = None, torch.ones(T, dtype=torch.float64)
    if scaled:
        scale = ops.RowScale((torch.rand(T, 130, generator=g) * 8).to(dev), 512, 1e-6)
        f = scale.factors().double().cpu()
    if bn == 0:
        bn, ctas = ops.gemm_swiglu_plan(I, K, dev)
        assert bn % 16 == 0 and ctas == -(-I // (bn // 2)) <= ops.num_sms(dev)
    out = torch.full((T, I), 7.0, device=dev, dtype=BF16)
    err = _err(dev)
    assert ops.gemm_bf16_swiglu(x, w, out, err, bn, row_scale=scale)
    assert int(err.item()) == 0
    y = (x.double().cpu() @ w.double().cpu().T) * f[:, None]
    gate, up = y[:, :I], y[:, I:]
    _close(out, gate / (1 + torch.exp(-gate)) * up, BF16)


# ------------------------------------------------------------------------ sampling
def _sample(dev, logits, temperature, top_k=0, top_p=1.0, u=0.0):
    from binfer_b200.csrc import ops
    R = logits.shape[0]
    f = lambda v, dt: torch.full((R,), v, dtype=dt, device=dev)
    uu = torch.as_tensor(u, dtype=torch.float32, device=dev).expand(R).contiguous()
    out = torch.empty(R, dtype=torch.int32, device=dev)
    ops.sample(logits, f(temperature, torch.float32), f(top_k, torch.int32),
               f(top_p, torch.float32), uu, out)
    return out.cpu().tolist()


def test_argmax_lowest_index_on_ties(cuda_device):
    logits = torch.randn(5, 3001, device=cuda_device)
    logits[0, [7, 2000, 2999]] = 50.0
    logits[1, 3000] = 50.0
    logits[2, 0] = 50.0
    logits[3] = 1.0                                   # all equal
    got = _sample(cuda_device, logits, 0.0)
    assert got[:4] == [7, 3000, 0, 0]
    assert got[4] == int(torch.argmax(logits[4]))


@pytest.mark.parametrize("temperature,top_k,top_p", [(0.8, 0, 1.0), (1.3, 5, 1.0), (0.7, 0, 0.6),
                                                     (1.0, 40, 0.9), (2.0, 1, 1.0)])
def test_sampling_matches_plain_sampler(cuda_device, temperature, top_k, top_p):
    g = torch.Generator().manual_seed(5)
    V = 1237
    logits = (3 * torch.randn(24, V, generator=g))
    us = torch.rand(24, generator=g)
    got = _sample(cuda_device, logits.to(cuda_device), temperature, top_k, top_p, us)
    for r in range(24):
        want = P.sample(logits[r], temperature, top_k, top_p, uniform=float(us[r]))
        if got[r] != want:
            # only a draw that lands within float rounding of a boundary may differ
            s = logits[r].double() / temperature
            p = torch.softmax(s, 0)
            cum = torch.cumsum(p, 0)
            assert abs(float(cum[min(got[r], want)]) - float(us[r])) < 1e-4, (r, got[r], want)


def test_top_k_confines_support_and_penalty(cuda_device):
    from binfer_b200.csrc import ops
    g = torch.Generator().manual_seed(1)
    logits = torch.randn(1, 500, generator=g)
    top = set(torch.topk(logits[0], 5).indices.tolist())
    dev_logits = logits.to(cuda_device).repeat(64, 1).contiguous()
    got = _sample(cuda_device, dev_logits, 1.5, top_k=5, u=torch.rand(64, generator=g))
    assert set(got) <= top and len(set(got)) > 1
    # repetition penalty flips the argmax (s > 0 ? s / pen : s * pen), twice for two occurrences
    lg = torch.tensor([[1.0, 3.0, 2.9, -1.0]], device=cuda_device)
    items = torch.tensor([[0, 1, 2], [0, 3, 1]], dtype=torch.int32, device=cuda_device)
    ops.repetition_penalty(lg, items, torch.tensor([1.5], device=cuda_device))
    assert torch.allclose(lg.cpu(), torch.tensor([[1.0, 3.0 / 2.25, 2.9, -1.5]]))
    assert _sample(cuda_device, lg, 0.0) == [2]


# ------------------------------------------------------------- tcgen05 matrix product
@pytest.mark.parametrize("M,N,K", [(1, 300, 200), (8, 128, 64), (7, 6144, 4096), (16, 4096, 4104),
                                   (33, 1000, 512), (64, 4096, 12288), (65, 272, 72),
                                   (128, 256, 64), (200, 700, 1000), (513, 2100, 2048)])
@pytest.mark.parametrize("out_dtype", [BF16, F32])
def test_gemm_bf16_tcgen05(cuda_device, M, N, K, out_dtype):
    """Token counts on both sides of the 128-row tile, widths and depths that are no
    multiple of the tile, bfloat16 and float32 results."""
    from binfer_b200.csrc import ops
    g = torch.Generator().manual_seed(M * 7 + N)
    x = torch.randn(M, K, generator=g).to(BF16).to(cuda_device)
    w = (0.05 * torch.randn(N, K, generator=g)).to(BF16).to(cuda_device)
    out = torch.full((M, N), 99.0, device=cuda_device, dtype=out_dtype)
    err = ops.error_word(cuda_device)
    assert ops.gemm_bf16(x, w, out, err)
    assert int(err.item()) == 0
    ref = x.double().cpu() @ w.double().cpu().T
    if out_dtype == BF16:
        _close(out, ref, BF16)
    else:
        # float accumulation of K products in the tensor core: error grows like sqrt(K)
        err_rel = float((out.double().cpu() - ref).abs().max() / ref.abs().max())
        assert err_rel <= 4e-7 * math.sqrt(K), err_rel
    # every tile width gives the same sums (one order of accumulation over K)
    for bn in (16, 48, 256):
        other = torch.empty_like(out)
        assert ops.gemm_bf16(x, w, other, err, bn=bn)
        assert torch.equal(other, out), f"tile width {bn} changes the result"


@pytest.mark.parametrize("M,N,K", [(1, 300, 200), (130, 128, 64), (256, 6144, 4096),
                                   (300, 1000, 520), (513, 2100, 2048), (700, 272, 72),
                                   (2048, 4096, 1024), (1000, 40, 4104)])
@pytest.mark.parametrize("out_dtype", [BF16, F32])
def test_gemm_bf16_pair(cuda_device, M, N, K, out_dtype):
    """The product on pairs of SMs: token counts on both sides of the 256-row tile and of a
    CTA's 128 rows, widths and depths that are no multiple of the tile, more tiles than pairs
    (the rings of stages and the two accumulators wrap), bfloat16 and float32 results."""
    from binfer_b200.csrc import ops
    g = torch.Generator().manual_seed(M * 7 + N)
    x = torch.randn(M, K, generator=g).to(BF16).to(cuda_device)
    w = (0.05 * torch.randn(N, K, generator=g)).to(BF16).to(cuda_device)
    out = torch.full((M, N), 99.0, device=cuda_device, dtype=out_dtype)
    err = ops.error_word(cuda_device)
    assert ops.gemm_bf16_pair(x, w, out, err)
    assert int(err.item()) == 0
    ref = x.double().cpu() @ w.double().cpu().T
    if out_dtype == BF16:
        _close(out, ref, BF16)
    else:
        err_rel = float((out.double().cpu() - ref).abs().max() / ref.abs().max())
        assert err_rel <= 4e-7 * math.sqrt(K), err_rel
    # every tile width gives the same sums (one order of accumulation over K); the narrow
    # ones leave by plain stores, multiples of 64 columns through shared memory and TMA stores
    for bn in (32, 160, 192, 256):
        other = torch.empty_like(out)
        assert ops.gemm_bf16_pair(x, w, other, err, bn=bn)
        assert torch.equal(other, out), f"tile width {bn} changes the result"
    assert int(err.item()) == 0


@pytest.mark.parametrize("M,N,K", [(5, 96, 64), (300, 1000, 520), (1024, 4096, 2048),
                                   (700, 2050, 72)])
def test_gemm_bf16_pair_adds_into_a_float_matrix(cuda_device, M, N, K):
    """``out += x w^T``: every element gets its sum once (through TMA reductions where the rows
    start on 16-byte boundaries, by plain read-add-write otherwise), rows and columns beyond
    the matrix are not touched, and a second call adds again."""
    from binfer_b200.csrc import ops
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn(M, K, generator=g).to(BF16).to(cuda_device)
    w = (0.05 * torch.randn(N, K, generator=g)).to(BF16).to(cuda_device)
    base = torch.randn(M + 3, N, generator=g).to(cuda_device)
    buf = base.clone()
    err = ops.error_word(cuda_device)
    assert ops.gemm_bf16_pair(x, w, buf[:M], err, accumulate=True)
    assert int(err.item()) == 0
    prod = x.double().cpu() @ w.double().cpu().T
    ref = base[:M].double().cpu() + prod
    got = buf[:M].double().cpu()
    assert float((got - ref).abs().max() / ref.abs().max()) <= 4e-7 * math.sqrt(K) + 1e-6
    assert torch.equal(buf[M:], base[M:])
    assert ops.gemm_bf16_pair(x, w, buf[:M], err, accumulate=True)
    ref2 = ref + prod
    assert float((buf[:M].double().cpu() - ref2).abs().max() / ref2.abs().max()) \
        <= 8e-7 * math.sqrt(K) + 1e-6
    assert int(err.item()) == 0


@pytest.mark.parametrize("M,I,K", [(3, 96, 64), (256, 12288, 1024), (300, 1000, 520),
                                   (1100, 3000, 2048), (129, 72, 4104), (2048, 1536, 4096)])
def test_gemm_bf16_pair_gated(cuda_device, M, I, K):
    """The stacked gate/up product with the activation in its epilogue: every output column
    pairs its gate row with the up row of the same output, at widths that are no multiple of
    the tile; the rows beyond a partial tile stay untouched."""
    from binfer_b200.csrc import ops
    g = torch.Generator().manual_seed(M + I)
    x = torch.randn(M, K, generator=g).to(BF16).to(cuda_device)
    w = (0.05 * torch.randn(2 * I, K, generator=g)).to(BF16).to(cuda_device)
    w[I:] *= torch.linspace(0.5, 2.0, I, device=cuda_device).to(BF16).unsqueeze(1)   # up rows differ
    buf = torch.full((M + 2, I), 99.0, device=cuda_device, dtype=BF16)
    out = buf[:M]
    err = ops.error_word(cuda_device)
    assert ops.gemm_bf16_pair(x, w, out, err, gated=True)
    assert int(err.item()) == 0
    gu = x.double().cpu() @ w.double().cpu().T
    ref = gu[:, :I] / (1 + torch.exp(-gu[:, :I])) * gu[:, I:]
    _close(out, ref, BF16)
    assert float(buf[M:].float().min()) == 99.0
    for bn in (64, 192, 256):
        other = torch.empty_like(out)
        assert ops.gemm_bf16_pair(x, w, other, err, bn=bn, gated=True)
        assert torch.equal(other, out), f"tile width {bn} changes the result"
    assert int(err.item()) == 0


def test_gemm_bf16_refuses_what_it_cannot_take(cuda_device):
    from binfer_b200.csrc import ops
    x = torch.randn(4, 100, device=cuda_device).to(BF16)       # K not a multiple of 8
    w = torch.randn(32, 100, device=cuda_device).to(BF16)
    out = torch.full((4, 32), 5.0, device=cuda_device, dtype=BF16)
    assert not ops.gemm_bf16(x, w, out, ops.error_word(cuda_device))
    assert bool((out == 5.0).all())


def test_engine_with_own_gemm_everywhere(cuda_device, tmp_path):
    """The bfloat16 engine with every product on the tcgen05 kernel still matches the plain
    implementation (config with hidden sizes that are multiples of 8)."""
    import helpers as H
    from binfer_b200.engine import make_env, make_runner, model_from_dir
    import importlib
    L = importlib.import_module("binfer_b200.parts.linear")
    d = H.make_model_dir(tmp_path, "B", BF16)
    raw, w = H.read_model_dir(d)
    reqs = {f"r{i}": H.random_tokens(n, raw["vocab_size"], n) for i, n in enumerate([70, 150, 9])}
    ref = {rid: P.forward(raw, w, t, torch.float64) for rid, t in reqs.items()}
    before = L._POLICY
    L.set_gemm_policy("own")
    try:
        env = make_env(BF16)
        steps = H.trace_mixed(reqs)
        runner = make_runner(model_from_dir(d, env), env, page_size=8,
                             num_pages=H.peak_pages(steps, 8))
        got = H.run_trace(runner, steps)
    finally:
        L.set_gemm_policy(before)
    worst = max(H.rel_err(row, ref[rid][p]) for (rid, p), row in got.items())
    assert worst <= 3e-2, worst


@pytest.mark.parametrize("nh,nkv,d,ps,window,spike", [
    (4, 2, 32, 16, None, False), (6, 1, 32, 8, None, True), (8, 2, 128, 16, None, True),
    (5, 5, 96, 4, 24, True), (3, 3, 64, 5, 70, True), (2, 1, 256, 16, 100, True),
    (4, 4, 128, 64, 130, True), (6, 2, 128, 8, None, True), (4, 1, 64, 32, 150, True)])
@pytest.mark.parametrize("variant", ["mma_sync", "umma", "umma2"])
def test_prefill_attention_over_pages(cuda_device, nh, nkv, d, ps, window, spike, variant):
    """Portions that start in the middle of a prompt, straddle 64-key tiles and pages, next to
    whole prompts; the far key and the window's edge are made to stand out."""
    from binfer_b200.csrc import ops
    if variant == "umma" and not (d in (64, 128) and ps >= 8 and 64 % ps == 0):
        pytest.skip("the umma variant does not take this head or page size")
    if variant == "umma2" and not (d == 128 and ps >= 8 and 64 % ps == 0):
        pytest.skip("the umma2 variant does not take this head or page size")
    ctxs, qlens = [70, 200, 129, 300, 64, 2, 400], [70, 37, 5, 130, 64, 2, 290]
    q, kc, vc, sot, pos, bt, ref = _attention_case(cuda_device, BF16, nh, nkv, d, ps, ctxs,
                                                   qlens, window, spike, seed=11)
    items, row = [], 0
    for b, (n, ql) in enumerate(zip(ctxs, qlens)):
        items.append([b, row, ql, n - ql])
        row += ql
    items = torch.tensor(items, dtype=torch.int32, device=cuda_device)
    out = torch.zeros_like(q)
    err = _err(cuda_device)
    ops.prefill_attention(q, kc, vc, items, len(ctxs), max(qlens), bt, out, nh, nkv, d, window,
                          d ** -0.5, err, variant=variant)
    assert int(err.item()) == 0
    _close(out, ref, BF16)
    # a subset of the portions leaves the other rows alone
    out2 = torch.zeros_like(q)
    ops.prefill_attention(q, kc, vc, items[1:3].contiguous(), 2, 37, bt, out2, nh, nkv, d,
                          window, d ** -0.5, err, variant=variant)
    assert torch.equal(out2[70:112], out[70:112]) and float(out2[:70].abs().max()) == 0.0


@pytest.mark.parametrize("splits", [2, 3, 8])
@pytest.mark.parametrize("ps,neighbours", [(16, True), (8, False), (64, False)])
def test_prefill_attention_keys_shared_out(cuda_device, splits, ps, neighbours):
    """Few queries after many cached keys: the keys of a block of 256 queries are shared out
    over several CTAs and merged.  Portions whose blocks have fewer key tiles than there are
    shares (an empty share), rows that see no key of a share (causal), a portion of two rows,
    and one from position 0, beside long prefixes; the far key is made to stand out."""
    from binfer_b200.csrc import ops
    nh, nkv, d = 4, 2, 128
    ctxs, qlens = [1500, 70, 2100, 2, 900], [200, 70, 300, 2, 129]
    q, kc, vc, sot, pos, bt, ref = _attention_case(cuda_device, BF16, nh, nkv, d, ps, ctxs,
                                                   qlens, None, True, seed=31,
                                                   neighbours=neighbours)
    items, row = [], 0
    for b, (n, ql) in enumerate(zip(ctxs, qlens)):
        items.append([b, row, ql, n - ql])
        row += ql
    items = torch.tensor(items, dtype=torch.int32, device=cuda_device)
    err = _err(cuda_device)
    out = torch.zeros_like(q)
    ops.prefill_attention(q, kc, vc, items, len(ctxs), max(qlens), bt, out, nh, nkv, d, None,
                          d ** -0.5, err, variant="umma2", splits=splits)
    assert int(err.item()) == 0
    _close(out, ref, BF16)
    # the number of shares chosen from the longest context gives the same values to rounding
    auto = torch.zeros_like(q)
    ops.prefill_attention(q, kc, vc, items, len(ctxs), max(qlens), bt, auto, nh, nkv, d, None,
                          d ** -0.5, err, max_ctx=max(ctxs))
    assert int(err.item()) == 0
    _close(auto, ref, BF16)


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6])
def test_prefill_attention_random_shapes(cuda_device, seed):
    """Shapes drawn at random (heads, groups, page size, window, how many portions, where they
    start and how long they are, pages side by side or scattered): the kernel that the policy
    picks, with the keys shared out or not as it decides, against the plain result."""
    import random
    from binfer_b200.csrc import ops
    rnd = random.Random(seed)
    nkv = rnd.choice([1, 2, 4])
    nh = nkv * rnd.choice([1, 2, 4, 7])
    d, ps = 128, rnd.choice([8, 16, 32, 64])
    window = rnd.choice([None, None, rnd.randint(40, 900)])
    n = rnd.randint(1, 4)
    qlens = [rnd.choice([2, rnd.randint(3, 130), rnd.randint(131, 700)]) for _ in range(n)]
    ctxs = [ql + rnd.choice([0, rnd.randint(1, 300), rnd.randint(1500, 3000)]) for ql in qlens]
    q, kc, vc, sot, pos, bt, ref = _attention_case(cuda_device, BF16, nh, nkv, d, ps, ctxs,
                                                   qlens, window, True, seed=100 + seed,
                                                   neighbours=rnd.random() < 0.5)
    items, row = [], 0
    for b, (c, ql) in enumerate(zip(ctxs, qlens)):
        items.append([b, row, ql, c - ql])
        row += ql
    items = torch.tensor(items, dtype=torch.int32, device=cuda_device)
    err = _err(cuda_device)
    out = torch.zeros_like(q)
    ops.prefill_attention(q, kc, vc, items, n, max(qlens), bt, out, nh, nkv, d, window,
                          d ** -0.5, err, max_ctx=max(ctxs))
    assert int(err.item()) == 0
    _close(out, ref, BF16)
    two = torch.zeros_like(q)
    ops.prefill_attention(q, kc, vc, items, n, max(qlens), bt, two, nh, nkv, d, window,
                          d ** -0.5, err, variant="umma2", splits=1)
    assert int(err.item()) == 0
    _close(two, ref, BF16)


@pytest.mark.parametrize("ps,window,neighbours", [(64, None, False), (16, 300, False),
                                                  (8, None, False), (16, None, True),
                                                  (8, 300, True), (32, 100, True)])
@pytest.mark.parametrize("variant", ["umma", "umma2"])
def test_prefill_attention_long_portions(cuda_device, ps, window, neighbours, variant):
    """Portions of many query tiles over many key tiles (the rings of stages wrap, the two
    query tiles of a block end on different key tiles), from the start of a prompt and from
    its middle, with and without a window; over shuffled pages and over pages that lie side
    by side in the pool, whose tiles come as one box (but for the tile a window cuts)."""
    from binfer_b200.csrc import ops
    nh, nkv, d = 4, 2, 128
    ctxs, qlens = [1500, 700, 1100], [900, 700, 257]
    q, kc, vc, sot, pos, bt, ref = _attention_case(cuda_device, BF16, nh, nkv, d, ps, ctxs,
                                                   qlens, window, True, seed=23,
                                                   neighbours=neighbours)
    items, row = [], 0
    for b, (n, ql) in enumerate(zip(ctxs, qlens)):
        items.append([b, row, ql, n - ql])
        row += ql
    items = torch.tensor(items, dtype=torch.int32, device=cuda_device)
    out = torch.zeros_like(q)
    err = _err(cuda_device)
    ops.prefill_attention(q, kc, vc, items, len(ctxs), max(qlens), bt, out, nh, nkv, d, window,
                          d ** -0.5, err, variant=variant)
    assert int(err.item()) == 0
    _close(out, ref, BF16)


@pytest.mark.parametrize("M,N,K,bn,c", [(1, 300, 520, 64, 4), (8, 4096, 4096, 128, 4),
                                        (16, 1000, 4104, 128, 8), (7, 6144, 4096, 192, 4),
                                        (3, 256, 256, 256, 2), (16, 4096, 12288, 128, 4),
                                        (5, 96, 64, 64, 4), (8, 24576, 4096, 176, 1),
                                        (2, 1000, 320, 80, 1), (17, 4096, 4096, 128, 4),
                                        (40, 520, 1024, 64, 2), (64, 4096, 12288, 128, 4),
                                        (33, 6144, 4096, 192, 4)])
@pytest.mark.parametrize("out_dtype", [BF16, F32])
def test_gemm_bf16_cluster_split_k(cuda_device, M, N, K, bn, c, out_dtype):
    """K split over a cluster and reduced through distributed shared memory; widths and depths
    that are no multiple of the tile, fewer K steps than CTAs in the cluster."""
    from binfer_b200.csrc import ops
    g = torch.Generator().manual_seed(M * 3 + N)
    x = torch.randn(M, K, generator=g).to(BF16).to(cuda_device)
    w = (0.05 * torch.randn(N, K, generator=g)).to(BF16).to(cuda_device)
    out = torch.full((M, N), 99.0, device=cuda_device, dtype=out_dtype)
    err = ops.error_word(cuda_device)
    assert ops.gemm_bf16_cluster(x, w, out, err, bn, c)
    assert int(err.item()) == 0
    ref = x.double().cpu() @ w.double().cpu().T
    if out_dtype == BF16:
        _close(out, ref, BF16)
    else:
        err_rel = float((out.double().cpu() - ref).abs().max() / ref.abs().max())
        assert err_rel <= 4e-7 * math.sqrt(K), err_rel
    again = torch.empty_like(out)
    assert ops.gemm_bf16_cluster(x, w, again, err, bn, c)
    assert torch.equal(again, out), "the split-K sum must have one fixed order"
    assert not ops.gemm_bf16_cluster(torch.zeros(65, K, device=cuda_device, dtype=BF16), w,
                                     torch.empty(65, N, device=cuda_device, dtype=out_dtype),
                                     err, bn, c)


@pytest.mark.parametrize("N,K,bn,c", [(5120, 25600, 192, 4), (5120, 8192, 192, 4)])
def test_gemm_bf16_cluster_many_k_steps_many_launches(cuda_device, N, K, bn, c):
    """A hundred K steps per CTA through a ring of seven slots, two issuing threads, a
    thousand launches: every launch gives the first one's bits and no wait gives up.  (Each
    ring slot has one issuer: were the K steps dealt out in turn, a thread would wait for
    every second fill of a slot with the same parity, which held only while the copies
    landed in order.  The Qwen3-32B shape's output and down projections are these sizes.)"""
    from binfer_b200.csrc import ops
    g = torch.Generator().manual_seed(N + K)
    x = torch.randn(8, K, generator=g).to(BF16).to(cuda_device)
    w = (0.05 * torch.randn(N, K, generator=g)).to(BF16).to(cuda_device)
    err = ops.error_word(cuda_device)
    first = torch.empty((8, N), device=cuda_device, dtype=BF16)
    assert ops.gemm_bf16_cluster(x, w, first, err, bn, c)
    _close(first, x.double().cpu() @ w.double().cpu().T, BF16)
    out = torch.empty_like(first)
    same = torch.ones((), dtype=torch.bool, device=cuda_device)
    for _ in range(1000):
        assert ops.gemm_bf16_cluster(x, w, out, err, bn, c)
        same &= (out == first).all()
    assert bool(same) and int(err.item()) == 0
