"""The kernels of the Dosovik layers alone against the plain functions: short convolution with its state, the norm
after the sum (and its fused forms), the preparation of attention rows, the polynomial activation, and attention
with a chunk mask and a sink on the plain and on the tensor-core kernels."""
import math

import pytest
import torch

import kernel_utils as K
import plain_dosovik as PD

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rts():
    from atoma_infer_b200.engine.runtime import make_runtime

    return {"bfloat16": make_runtime("bfloat16", "cuda:0"), "float32": make_runtime("float32", "cuda:0")}


def _tables(entries, page):
    return K.scrambled_tables([c + n for c, n in entries], page, seed=1)


@pytest.mark.parametrize("taps,C", [(4, 96), (2, 40), (5, 1100), (1, 64)])
def test_short_conv_over_portions_and_slots(rts, taps, C):
    """Three requests fed in portions of 1 to 9 rows, in one batch, their states in slots that are slices of a wider
    per-request state; every portion's output equals the plain convolution of the whole sequence."""
    rt = rts["float32"]
    ops = rt.ops
    g = torch.Generator().manual_seed(taps)
    lens = [23, 9, 14]
    xs = [torch.randn(n, C, generator=g) for n in lens]
    w = torch.randn(C, taps, generator=g)
    want = [x + PD.short_conv(x.double(), w.double()).float() for x in xs]
    R = taps - 1
    wide = torch.full((3, 7 + R * C + 5), float("nan"), device=rt.device)  # NaN: a row read before it was written shows
    state = wide[:, 7:7 + R * C].unflatten(1, (R, C)) if R else None
    wd = w.t().contiguous().to(rt.device)  # the kernels take [taps, channels]
    at = [0, 0, 0]
    sizes = [1, 2, 9, 3, 1, 1, 4, 2]
    step = 0
    while any(a < n for a, n in zip(at, lens)):
        entries, rows = [], []
        for k in range(3):
            n = min(sizes[(step + k) % len(sizes)], lens[k] - at[k])
            entries.append((at[k], n))
            rows.append(xs[k][at[k]:at[k] + n])
        live = [k for k in range(3) if entries[k][1] > 0]
        # entries of the step are the live requests; their slots are their request numbers
        ctx, _ = K.make_context(rt, [entries[k] for k in live], 16, [[1]] * len(live))
        ctx.state_slots.copy_(torch.tensor(live, dtype=torch.int32))
        x = torch.cat([rows[k] for k in live]).to(rt.device)
        for dtype in (torch.float32, torch.bfloat16):
            out = torch.empty((ctx.T, C), dtype=dtype, device=rt.device)
            ops.short_conv(x, wd, state, ctx, out)
            r = 0
            for k in live:
                n = entries[k][1]
                exp = want[k][at[k]:at[k] + n]
                tol = 1e-5 if dtype == torch.float32 else 2e-2
                assert torch.allclose(out[r:r + n].float().cpu(), exp, atol=tol * float(exp.abs().max())), (step, k, dtype)
                r += n
        ops.short_conv_save(x, state, ctx, taps)
        for k in live:
            at[k] += entries[k][1]
        step += 1
    ops.check_status()


@pytest.mark.parametrize("H,alpha", [(96, 3.0), (1000, 1.0), (2048, 0.5)])
def test_norm_after_the_sum(rts, H, alpha):
    rt = rts["float32"]
    g = torch.Generator().manual_seed(H)
    entries = [(0, 5), (7, 1), (3, 2)]
    ctx, _ = K.make_context(rt, entries, 16, [[1]] * 3)
    x, d, w = torch.randn(ctx.T, H, generator=g), torch.randn(ctx.T, H, generator=g), 1 + 0.2 * torch.randn(H, generator=g)
    want = PD.rms_divide(alpha * x.double() + d.double(), 1e-5) * w.double()
    for dd in (d, d.bfloat16()):
        resid = x.clone().to(rt.device)
        rt.ops.scaled_add_rmsnorm(resid, dd.to(rt.device), alpha, w.to(rt.device), 1e-5, ctx)
        ref = PD.rms_divide(alpha * x.double() + dd.double(), 1e-5) * w.double()
        assert torch.allclose(resid.cpu().double(), ref, atol=2e-6 * float(want.abs().max()))
    # keep: the rows as they were go to the ring of a convolution (the last taps - 1 rows of every entry, by position)
    taps = 3
    state = torch.full((3, taps - 1, H), float("nan"), device=rt.device)
    resid = x.clone().to(rt.device)
    rt.ops.scaled_add_rmsnorm(resid, d.to(rt.device), alpha, w.to(rt.device), 1e-5, ctx, keep=(state, taps))
    assert torch.equal(state[0, 3 % 2].cpu(), x[3]) and torch.equal(state[0, 4 % 2].cpu(), x[4])
    assert torch.equal(state[1, 7 % 2].cpu(), x[5]) and torch.isnan(state[1, 0]).all()
    assert torch.equal(state[2, 3 % 2].cpu(), x[6]) and torch.equal(state[2, 4 % 2].cpu(), x[7])


def test_norm_after_the_sum_leaves_the_next_input_in_decode_steps(rts):
    """Decode steps: the norm kernel also writes new row + conv(new row, state); the same as the two kernels apart."""
    rt = rts["float32"]
    g = torch.Generator().manual_seed(3)
    H, taps = 160, 4
    entries = [(0, 1), (1, 1), (2, 1), (9, 1)]  # the first positions of a request: rows before its start are zeros
    ctx, _ = K.make_context(rt, entries, 16, [[1]] * 4)
    x, d = torch.randn(4, H, generator=g).to(rt.device), torch.randn(4, H, generator=g).to(rt.device)
    w, cw = (1 + 0.1 * torch.randn(H, generator=g)).to(rt.device), torch.randn(taps, H, generator=g).to(rt.device)
    state = torch.randn(4, taps - 1, H, generator=g).to(rt.device)
    for dtype in (torch.float32, torch.bfloat16):
        a, b = x.clone(), x.clone()
        fused = torch.empty((4, H), dtype=dtype, device=rt.device)
        rt.ops.scaled_add_rmsnorm(a, d, 2.0, w, 1e-6, ctx, conv=(cw, state, fused))
        rt.ops.scaled_add_rmsnorm(b, d, 2.0, w, 1e-6, ctx)
        apart = torch.empty((4, H), dtype=dtype, device=rt.device)
        rt.ops.short_conv(b, cw, state, ctx, apart)
        assert torch.equal(a, b)
        assert torch.allclose(fused.float(), apart.float(), atol=1e-5 if dtype == torch.float32 else 2e-2)
    # position 0 sees only itself, whatever the ring holds
    want0 = b[0] * (1 + cw[taps - 1])
    assert torch.allclose(apart[0].float(), want0, atol=3e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("entries", [[(0, 5), (13, 3), (40, 1)], [(3, 2100), (0, 7)]])  # thousands of rows: several a block
@pytest.mark.parametrize("nq,nkv,d,dv,rot", [(4, 2, 48, 32, 48), (6, 2, 24, 16, 8), (4, 4, 16, 32, 16), (2, 1, 64, 64, 32), (3, 1, 40, 40, 0),
                                             (2, 2, 18, 10, 6)])  # the last: sizes that are no multiples of 4
def test_attention_rows_are_prepared(rts, dtype, entries, nq, nkv, d, dv, rot):
    rt = rts[dtype]
    g = torch.Generator().manual_seed(d + dv)
    page, dp = 8, -(-max(d, dv) // 16) * 16
    tables, num_pages = _tables(entries, page)
    ctx, _ = K.make_context(rt, entries, page, tables)
    T, NQ, NK, NV = ctx.T, nq * d, nkv * d, nkv * dv
    qkv = torch.randn(T, NQ + NK + NV, generator=g).to(rt.dtype)
    # values that bfloat16 holds exactly: the kernel takes them in float32 or, beside bfloat16 rows, as they are stored
    bias = torch.randn(NQ + NK + NV, generator=g).bfloat16().float()
    qn, kn = (1 + 0.3 * torch.randn(NQ, generator=g)).bfloat16().float(), (1 + 0.3 * torch.randn(NK, generator=g)).bfloat16().float()
    stored = rt.dtype if rot % 16 == 0 else torch.float32
    v_first, lam = torch.randn(T, NV, generator=g).to(rt.dtype), torch.tensor([0.37])
    inv_freq = (100.0 ** (-torch.arange(0, rot, 2, dtype=torch.float64) / rot)).float() if rot else None
    cache = torch.full((num_pages, 2, nkv, page, dp), float("nan"), dtype=rt.dtype, device=rt.device)
    q_out = torch.full((T, nq * dp), float("nan"), dtype=rt.dtype, device=rt.device)
    v_out = torch.empty((T, NV), dtype=rt.dtype, device=rt.device)
    dev = lambda t: t.to(rt.device) if t is not None else None  # noqa: E731
    rt.ops.qkv_prepare(dev(qkv), ctx, cache, 0, q_out, nq=nq, nkv=nkv, d=d, dv=dv, dp=dp, page_size=page, num_pages=num_pages,
                       store_kv=True, bias=dev(bias.to(stored)), q_norm=dev(qn.to(stored)), k_norm=dev(kn.to(stored)), eps=1e-5, inv_freq=dev(inv_freq), rot=rot,
                       v_first=dev(v_first), v_lambda=dev(lam), v_out=v_out)
    rt.ops.check_status()
    rows = qkv.double() + bias.double()
    pos = torch.cat([torch.arange(c, c + n) for c, n in entries])
    q = (PD.rms_divide(rows[:, :NQ], 1e-5) * qn.double()).view(T, nq, d)
    k = (PD.rms_divide(rows[:, NQ:NQ + NK], 1e-5) * kn.double()).view(T, nkv, d)
    if rot:
        q, k = PD.partial_rotation(q, pos, rot, 100.0), PD.partial_rotation(k, pos, rot, 100.0)
    v = rows[:, NQ + NK:]
    vm = ((1 - 0.37) * v + 0.37 * v_first.double()).view(T, nkv, dv)
    # angles are position x frequency in float32: their rounding grows with the position
    tol = (1e-5 + 2e-7 * max(c + n for c, n in entries)) if dtype == "float32" else 2e-2
    got_q = q_out.float().cpu().view(T, nq, dp)
    assert torch.allclose(got_q[..., :d].double(), q, atol=tol * float(q.abs().max())) and (got_q[..., d:] == 0).all()
    assert torch.allclose(v_out.float().cpu().double(), v, atol=tol * float(v.abs().max()))
    row = 0
    for (c, n), table in zip(entries, tables):
        for p in range(c, c + n):
            kk, vv = (cache[table[p // page], i, :, p % page].float().cpu() for i in (0, 1))
            assert torch.allclose(kk[:, :d].double(), k[row], atol=tol * float(k.abs().max())) and (kk[:, d:] == 0).all()
            assert torch.allclose(vv[:, :dv].double(), vm[row], atol=tol * float(vm.abs().max())) and (vv[:, dv:] == 0).all()
            row += 1


@pytest.mark.parametrize("F", [320, 1000, 4096])
def test_polynomial_activation(rts, F):
    g = torch.Generator().manual_seed(F)
    coef = torch.tensor([0.7, -0.4, 0.25, 0.1])
    for dtype in ("float32", "bfloat16"):
        rt = rts[dtype]
        z = (2.0 * torch.randn(5, F, generator=g)).to(rt.dtype)
        out = torch.empty_like(z, device=rt.device)
        rt.ops.polynorm(z.to(rt.device), coef.to(rt.device), 1e-6, out, None)
        want = PD.poly_norm(z.double(), coef.double(), 1e-6)
        assert torch.allclose(out.float().cpu().double(), want, atol=(1e-5 if dtype == "float32" else 1.5e-2) * float(want.abs().max()))


def _chunk_sink_case(rt, entries, nq, nkv, d, page, chunk, sink, seed=0, stand_out=None, splits=None, fast=True):
    """Attention of a step over a hand-filled cache; returns the largest difference from the plain attention."""
    g = torch.Generator().manual_seed(seed)
    lengths = [c + n for c, n in entries]
    tables, num_pages = K.scrambled_tables(lengths, page, seed)
    qs, ks, vs = ([torch.randn(L, h, d, generator=g) for L in lengths] for h in (nq, nkv, nkv))
    if stand_out is not None:  # (key, query): that key towers for that query, if the query may see it
        for q, k, (key, qi) in zip(qs, ks, stand_out):
            k[key] *= 3.0
            q[qi] = k[key].repeat_interleave(nq // nkv, dim=0) * 1.5
    qs, ks, vs = ([t.to(rt.dtype).float() for t in x] for x in (qs, ks, vs))
    cache = torch.full((num_pages, 2, nkv, page, d), float("nan"), dtype=rt.dtype, device=rt.device)
    K.fill_cache(cache, tables, ks, vs, page)
    ctx, _ = K.make_context(rt, entries, page, tables)
    q = torch.cat([x[c:c + n].reshape(n, nq * d) for (c, n), x in zip(entries, qs)]).to(rt.dtype).to(rt.device)
    out = torch.full((ctx.T, nq * d), float("nan"), dtype=rt.dtype, device=rt.device)
    ops = rt.ops
    ops.masked_fast_attention = fast
    if splits is not None:
        ops.decode_splits = lambda *a: splits
    try:
        ops.attention(q, nq * d, cache, ctx, 0, out, nq, nkv, d, page, num_pages, 0, 1 / math.sqrt(d), chunk=chunk, sink=sink)
    finally:
        ops.masked_fast_attention = True
        if splits is not None:
            del ops.decode_splits
    ops.check_status()
    worst, row = 0.0, 0
    for (c, n), qq, k, v in zip(entries, qs, ks, vs):
        plain = lambda vals: PD.chunk_sink_attention(qq.double(), k.double(), vals.double(), 1 / math.sqrt(d), chunk or None,  # noqa: E731
                                                     rows=range(c, c + n))[c:c + n]
        want = plain(v)
        if not sink:  # without a sink: the same with the sink's share given back
            want = want / plain(torch.ones_like(v))
        worst = max(worst, float((out[row:row + n].float().cpu().view(n, nq, d).double() - want).abs().max()))
        row += n
    return worst


@pytest.mark.parametrize("dtype,fast", [("float32", True), ("bfloat16", True), ("bfloat16", False)])
@pytest.mark.parametrize("d,nq,nkv,page,chunk", [(48, 4, 2, 16, 120), (64, 4, 1, 8, 64), (32, 6, 3, 4, 21), (128, 2, 2, 16, 100)])
def test_chunks_and_sink_in_prompt_portions(rts, dtype, fast, d, nq, nkv, page, chunk):
    """Portions that start and end inside chunks, cross one or several chunk edges, and sit beside single tokens; for
    the last query of each request one key towers: the newest key outside its chunk, or the oldest inside."""
    rt = rts[dtype]
    tol = 2e-5 if dtype == "float32" else 2.5e-2
    entries = [(0, 3 * chunk + 5), (chunk - 2, 7), (2 * chunk - 1, 1), (chunk + 3, 2), (5, 2 * chunk)]
    for which in ("outside", "inside"):
        marks = []
        for c, n in entries:
            last = c + n - 1
            start = last - last % chunk
            marks.append((max(start - 1, 0) if which == "outside" else start, last))
        for sink in (True, False):
            # head sizes 64 and 128 with pages of 8 and more: the tcgen05 kernel, and the mma.sync kernel in its place
            for tc in ((True, False) if dtype == "bfloat16" and fast and d in (64, 128) else (True,)):
                rt.ops.tc_attention = tc
                try:
                    err = _chunk_sink_case(rt, entries, nq, nkv, d, page, chunk, sink, seed=chunk, stand_out=marks, fast=fast)
                finally:
                    rt.ops.tc_attention = True
                assert err < tol, (which, sink, tc, err)


@pytest.mark.parametrize("dtype,fast", [("float32", True), ("bfloat16", True), ("bfloat16", False)])
@pytest.mark.parametrize("d,nq,nkv,page,chunk,splits", [(48, 4, 2, 16, 120, None), (64, 8, 1, 8, 512, 4), (64, 8, 1, 8, 3000, 12),
                                                         (32, 6, 3, 4, 21, 2), (128, 4, 2, 16, 0, 3)])
def test_chunks_and_sink_in_decode_steps(rts, dtype, fast, d, nq, nkv, page, chunk, splits):
    """Every request brings one token: at the first and last position of a chunk, one past an edge, deep inside a
    long chunk (split key ranges, merged in a cluster and through scratch), and at the start of a sequence."""
    rt = rts[dtype]
    tol = 2e-5 if dtype == "float32" else 2.5e-2
    c = chunk or 700
    ctxs = [0, 1, c - 1, c, c + 1, 2 * c - 1, 2 * c + c // 2, c // 2]
    entries = [(p, 1) for p in ctxs]
    for which in ("outside", "inside"):
        marks = []
        for p, _ in entries:
            start = p - p % chunk if chunk else 0
            marks.append((max(start - 1, 0) if which == "outside" else start, p))
        for sink in (True, False):
            err = _chunk_sink_case(rt, entries, nq, nkv, d, page, chunk, sink, seed=c, stand_out=marks, splits=splits, fast=fast)
            assert err < tol, (which, sink, err)
