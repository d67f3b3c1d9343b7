"""The kernels of the Tutezen layers alone against the plain functions: the pending sum with its norm, the causal
convolution with bias and SiLU and its ring, the state-space recurrence in order and in chunks of time, the gated norm
in parts, the norm over a slice, linears per head, the rows of latent attention, a window and a learned sink on the
plain and on the tensor-core attention kernels, the router and the experts."""
import math

import pytest
import torch

import kernel_utils as K
import plain_tutezen as PT
from atoma_infer_b200.parts.base import PendingSum

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rts():
    from atoma_infer_b200.engine.runtime import make_runtime

    return {"bfloat16": make_runtime("bfloat16", "cuda:0"), "float32": make_runtime("float32", "cuda:0")}


def _tables(entries, page):
    return K.scrambled_tables([c + n for c, n in entries], page, seed=1)


def _err(got, want):
    return float((got.double().cpu() - want.double()).abs().max()) / max(float(want.abs().max()), 1e-9)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H", [96, 1100, 90])  # (90: rows that do not start on 16 bytes, one value a thread and step)
def test_pending_sum_and_norm(rts, dtype, H):
    rt = rts[dtype]
    entries = [(0, 5), (3, 1), (7, 4)]
    tables, _ = _tables(entries, 4)
    ctx, rows = K.make_context(rt, entries, 4, tables, rows=[9, 0, 4])
    g = torch.Generator().manual_seed(H)
    resid0 = torch.randn(10, H, generator=g)
    a, b = (torch.randn(10, H, generator=g).to(rt.dtype) for _ in range(2))
    more, vec, w = torch.randn(10, H, generator=g), torch.randn(H, generator=g), torch.rand(H, generator=g) + 0.5
    dev = lambda t: t.to(rt.device)  # noqa: E731
    for terms, extra in (((a, b), True), ((a,), False), ((), True)):
        want = resid0.double() + 0.3 * sum((t.double() for t in terms), torch.zeros(10, H, dtype=torch.float64))
        if extra:
            want = want + more.double() + vec.double()
        pend = PendingSum(tuple(dev(t) for t in terms), 0.3, dev(more) if extra else None, dev(vec) if extra else None)
        resid = dev(resid0.clone())
        out = torch.empty(10, H, dtype=rt.dtype, device=rt.device)
        rt.ops.sum_rmsnorm(resid, pend, dev(w), 1e-5, out, ctx.meta, ctx.T)
        assert _err(resid, want) < 1e-6
        assert _err(out, PT.rms_divide(want, 1e-5) * w.double()) < (1e-5 if dtype == "float32" else 1e-2)
        resid = dev(resid0.clone())  # at gathered rows the stream stays as it is
        out3 = torch.empty(3, H, dtype=rt.dtype, device=rt.device)
        rt.ops.sum_rmsnorm(resid, pend, dev(w), 1e-5, out3, ctx.meta, 3, rows=rows)
        assert torch.equal(resid.cpu(), resid0) and torch.equal(out3.cpu(), out.cpu()[[9, 0, 4]])
        resid = dev(resid0.clone())  # and without a norm only the sum is taken
        rt.ops.sum_rmsnorm(resid, pend, None, 0.0, None, ctx.meta, ctx.T)
        assert _err(resid, want) < 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("pad", [7, 8])
@pytest.mark.parametrize("taps,C", [(4, 96), (2, 40), (5, 1100), (1, 64)])
def test_convolution_over_portions_and_slots(rts, dtype, taps, C, pad):
    """Three requests fed in portions of 1 to 9 rows in one batch, the input a slice of wider rows, the rings slices of a
    wider per-request state (whose width lets the kernel take several channels a thread, or not); every portion's output
    equals the plain convolution of the whole sequence.  Towards the end every request brings one row, and the
    convolution updates the ring itself."""
    rt = rts[dtype]
    g = torch.Generator().manual_seed(taps * 1000 + C)
    lengths, wide = (23, 9, 17), C + 24
    seqs = [torch.randn(n, wide, generator=g).to(rt.dtype) for n in lengths]
    w, b = torch.randn(C, taps, generator=g), torch.randn(C, generator=g)
    want = [PT.silu(PT.causal_conv(s[:, 8:8 + C].double(), w.double(), b.double())) for s in seqs]
    state = torch.full((3, (taps - 1) * C + pad), float("nan"), device=rt.device)
    ring = state[:, 4:4 + (taps - 1) * C].view(3, taps - 1, C) if taps > 1 else None
    wt, bd = w.t().contiguous().to(rt.device), b.to(rt.device)
    pos, cuts, step = [0, 0, 0], (1, 5, 2, 9, 3, 4, 1, 1, 1, 1, 1, 1, 1, 1, 1), 0
    while any(p < n for p, n in zip(pos, lengths)):
        entries, parts, who = [], [], []
        for k, n in enumerate(lengths):
            if pos[k] >= n:
                continue
            take = min(cuts[(step + k) % len(cuts)], n - pos[k])
            entries.append((pos[k], take))
            parts.append(seqs[k][pos[k]:pos[k] + take])
            who.append(k)
        tables, _ = _tables(entries, 4)
        ctx, _ = K.make_context(rt, entries, 4, tables)
        ctx.state_slots.copy_(torch.tensor(who, dtype=torch.int32))
        rows = torch.cat(parts).to(rt.device)
        out = torch.full((ctx.T, C), float("nan"), dtype=rt.dtype, device=rt.device)
        if not rt.ops.causal_conv_act(rows[:, 8:8 + C], wt, bd, ring, ctx, out, act="silu"):
            rt.ops.causal_conv_save(rows[:, 8:8 + C], ring, ctx, taps)
        at = 0
        for k, (c, n) in zip(who, entries):
            assert _err(out[at:at + n], want[k][c:c + n]) < (1e-5 if dtype == "float32" else 1e-2), (step, k)
            at += n
            pos[k] += n
        step += 1
    rt.ops.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,P,N,G", [(3, 16, 24, 1), (4, 8, 40, 2), (2, 64, 128, 2), (8, 24, 16, 4), (2, 32, 200, 1), (2, 12, 20, 1)])
def test_recurrence_in_order_and_in_chunks(rts, dtype, heads, P, N, G):
    """Portions of 1 to 300 tokens beside each other (the long ones run as chunks of time side by side), states in slots
    of a wider per-request state, twice over the same slots: the state is carried, and nothing depends on the cut."""
    rt = rts[dtype]
    g = torch.Generator().manual_seed(heads * 100 + N)
    inner = heads * P
    lengths = (341, 7, 130)
    xbc = [(torch.randn(n, inner + 2 * G * N, generator=g) * 0.7).to(rt.dtype) for n in lengths]
    dt = [(torch.randn(n, heads + 3, generator=g) * 2 - 1).to(rt.dtype) for n in lengths]
    dt_bias, a_log, d = torch.randn(heads, generator=g), torch.randn(heads, generator=g) * 0.5 - 1.0, torch.randn(heads, generator=g)
    want = []
    for s, r in zip(xbc, dt):
        s, step = s.double(), PT.softplus(r[:, 2:2 + heads].double() + dt_bias.double())
        want.append(PT.state_space(s[:, :inner].reshape(-1, heads, P), s[:, inner:inner + G * N].reshape(-1, G, N),
                                   s[:, inner + G * N:].reshape(-1, G, N), step, a_log.double(), d.double(), G).reshape(-1, inner))
    state = torch.zeros((3, heads * N * P + 5), device=rt.device)
    mats = state[:, 4:4 + heads * N * P].view(3, heads, N, P)
    assert mats.stride(0) == heads * N * P + 5
    dev = lambda t: t.to(rt.device)  # noqa: E731
    for cuts in ((300, 1, 40), (2, 3, 129)):   # then the rest
        pos = [0, 0, 0]
        for _ in range(2):
            entries = [(pos[k], min(cuts[k], lengths[k] - pos[k]) if _ == 0 else lengths[k] - pos[k]) for k in range(3)]
            who = [k for k in range(3) if entries[k][1] > 0]
            entries = [entries[k] for k in who]
            tables, _t = _tables(entries, 4)
            ctx, _r = K.make_context(rt, entries, 4, tables)
            ctx.state_slots.copy_(torch.tensor(who, dtype=torch.int32))
            rows = dev(torch.cat([xbc[k][c:c + n] for k, (c, n) in zip(who, entries)]))
            steps = dev(torch.cat([dt[k][c:c + n] for k, (c, n) in zip(who, entries)]))
            y = torch.full((ctx.T, inner), float("nan"), device=rt.device)
            rt.ops.ssm_scan(rows, steps[:, 2:2 + heads], dev(dt_bias), dev(a_log), dev(d), mats, ctx, y, heads=heads, head_dim=P,
                            nstate=N, groups=G)
            at = 0
            for k, (c, n) in zip(who, entries):
                assert _err(y[at:at + n], want[k][c:c + n]) < 2e-5, (cuts, k, c, n)
                at += n
                pos[k] += n
        mats.zero_()
    rt.ops.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,parts", [(48, 3), (32, 1), (1280, 2), (30, 3), (9000, 1)])
def test_gated_norm_in_parts(rts, dtype, n, parts):
    rt = rts[dtype]
    g = torch.Generator().manual_seed(n)
    entries = [(0, 6), (2, 1)]
    ctx, _ = K.make_context(rt, entries, 4, _tables(entries, 4)[0])
    y, z, w = torch.randn(7, n, generator=g), torch.randn(7, n + 9, generator=g).to(rt.dtype), torch.rand(n, generator=g) + 0.5
    out = torch.empty(7, n, dtype=rt.dtype, device=rt.device)
    rt.ops.gated_group_norm(y.to(rt.device), z.to(rt.device)[:, 5:5 + n], w.to(rt.device), parts, 1e-5, out, ctx.meta)
    want = PT.grouped_rms(y.double() * PT.silu(z[:, 5:5 + n].double()), parts, 1e-5) * w.double()
    assert _err(out, want) < (1e-5 if dtype == "float32" else 1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_over_a_slice_and_linears_per_head(rts, dtype):
    rt = rts[dtype]
    tol = 1e-5 if dtype == "float32" else 1.5e-2
    g = torch.Generator().manual_seed(3)
    for T in (5, 70):  # few rows: the own kernel; many rows in bfloat16: a batched library product
        entries = [(0, T - 1), (4, 1)]
        ctx, _ = K.make_context(rt, entries, 4, _tables(entries, 4)[0])
        x = torch.randn(T, 100, generator=g).to(rt.dtype)
        w = torch.rand(40, generator=g) + 0.5
        out = torch.empty(T, 40, dtype=rt.dtype, device=rt.device)
        rt.ops.rms_rows(x.to(rt.device)[:, 30:70], w.to(rt.device), 1e-6, out, ctx.meta)
        assert _err(out, PT.rms_divide(x[:, 30:70].double(), 1e-6) * w.double()) < tol
        for heads, Kd, N in ((3, 20, 48), (5, 130, 24)):
            xs = torch.randn(T, heads, Kd + 6, generator=g).to(rt.dtype)
            wh = (torch.randn(heads, N, Kd, generator=g) / math.sqrt(Kd)).to(rt.dtype)
            gate = torch.randn(T, heads * N + 11, generator=g).to(rt.dtype)
            want = torch.einsum("thk,hnk->thn", xs[:, :, 2:2 + Kd].double(), wh.double())
            out = torch.empty(T, heads, N, dtype=rt.dtype, device=rt.device)
            rt.ops.head_linear(xs.to(rt.device)[:, :, 2:2 + Kd], wh.to(rt.device), out, ctx.meta)
            assert _err(out, want) < tol
            gv = gate[:, 11:].view(T, heads, N)
            rt.ops.head_linear(xs.to(rt.device)[:, :, 2:2 + Kd], wh.to(rt.device), out, ctx.meta,
                               gate=gate.to(rt.device)[:, 11:].view(T, heads, N))
            assert _err(out, want * torch.sigmoid(gv.double())) < tol
    rt.ops.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,rank,rdim,rot,page", [(3, 48, 8, 8, 4), (2, 20, 16, 6, 8), (5, 32, 16, 0, 16), (2, 21, 10, 4, 4)])
def test_latent_rows(rts, dtype, heads, rank, rdim, rot, page):
    """Queries laid out for the attention kernels, the cached vector on both planes of its page, zeros behind both; the
    rotation pairs neighbours, of the first `rot` rotated dimensions only."""
    rt = rts[dtype]
    tol = 1e-5 if dtype == "float32" else 1e-2
    g = torch.Generator().manual_seed(rank)
    D = -(-(rank + rdim) // 16) * 16
    entries = [(0, 6), (37, 1), (5, 3)] if rank != 32 else [(0, 600), (37, 1), (5, 3)]  # (many tokens: a token a block)
    tables, num_pages = _tables(entries, page)
    ctx, _ = K.make_context(rt, entries, page, tables)
    T = ctx.T
    q = torch.randn(T, heads, 12 + rdim, generator=g).to(rt.dtype)
    q_abs = torch.randn(T, heads, rank, generator=g).to(rt.dtype)
    dkv = torch.randn(T, 7 + rank + rdim, generator=g).to(rt.dtype)
    w = torch.rand(rank, generator=g) + 0.5
    inv_freq = (1e4 ** (-torch.arange(0, rot, 2, dtype=torch.float64) / max(rot, 1))).float() if rot else None
    cache = torch.full((num_pages, 2, 1, page, D), float("nan"), dtype=rt.dtype, device=rt.device)
    q_out = torch.full((T, heads * D), float("nan"), dtype=rt.dtype, device=rt.device)
    dev = lambda t: t.to(rt.device) if t is not None else None  # noqa: E731
    rt.ops.latent_rows(dev(q)[:, :, 12:], dev(q_abs), dev(dkv)[:, 7:], dev(w), 1e-5, ctx, cache, 0, q_out, heads=heads, kv_rank=rank,
                       rot_dim=rdim, padded=D, page_size=page, num_pages=num_pages, store=True, inv_freq=dev(inv_freq), rotary_dims=rot)
    rt.ops.check_status()
    pos = torch.cat([torch.arange(c, c + n) for c, n in entries])
    turn = (lambda v: PT.rotate_pairs(v.double(), pos, rot, 1e4)) if rot else (lambda v: v.double())  # noqa: E731
    want_q = torch.zeros(T, heads, D, dtype=torch.float64)
    want_q[..., :rank], want_q[..., rank:rank + rdim] = q_abs.double(), turn(q[:, :, 12:])
    assert _err(q_out.view(T, heads, D), want_q) < tol
    key = torch.zeros(T, D, dtype=torch.float64)
    key[:, :rank] = PT.rms_divide(dkv[:, 7:7 + rank].double(), 1e-5) * w.double()
    key[:, rank:rank + rdim] = turn(dkv[:, 7 + rank:])
    t = 0
    for k, (c, n) in enumerate(entries):
        for p in range(c, c + n):
            for plane in (0, 1):
                assert _err(cache[tables[k][p // page], plane, 0, p % page], key[t]) < tol
            t += 1


def _window_sink_case(rt, entries, nq, d, page, window, sinks, seed=0, stand_out=None, splits=None, fast=True):
    """Attention of a step over a hand-filled cache with one key/value head whose values are its keys; returns the
    largest difference from the plain softmax with a window and a learned sink per head, as a share of the largest value
    (the values are the keys, and a towering key is several times larger than the rest)."""
    g = torch.Generator().manual_seed(seed)
    lengths = [c + n for c, n in entries]
    tables, num_pages = K.scrambled_tables(lengths, page, seed)
    qs = [torch.randn(L, nq, d, generator=g) for L in lengths]
    ks = [torch.randn(L, 1, d, generator=g) for L in lengths]
    if stand_out is not None:  # (key, query): that key towers for that query, if the query may see it
        for q, k, (key, qi) in zip(qs, ks, stand_out):
            k[key] *= 3.0
            q[qi] = k[key].repeat_interleave(nq, dim=0) * 1.5
    qs, ks = ([t.to(rt.dtype).float() for t in x] for x in (qs, ks))
    cache = torch.full((num_pages, 2, 1, page, d), float("nan"), dtype=rt.dtype, device=rt.device)
    K.fill_cache(cache, tables, ks, ks, page)
    ctx, _ = K.make_context(rt, entries, page, tables)
    q = torch.cat([x[c:c + n].reshape(n, nq * d) for (c, n), x in zip(entries, qs)]).to(rt.dtype).to(rt.device)
    out = torch.full((ctx.T, nq * d), float("nan"), dtype=rt.dtype, device=rt.device)
    ops = rt.ops
    ops.masked_fast_attention = fast
    if splits is not None:
        ops.decode_splits = lambda *a: splits
    scale = 1 / math.sqrt(d)
    try:
        ops.attention(q, nq * d, cache, ctx, 0, out, nq, 1, d, page, num_pages, window, scale, sink=sinks.to(rt.device))
    finally:
        ops.masked_fast_attention = True
        if splits is not None:
            del ops.decode_splits
    ops.check_status()
    worst, row, top = 0.0, 0, 1.0
    for (c, n), qq, k in zip(entries, qs, ks):
        for h in range(nq):
            p = PT.windowed_sink_softmax((qq[:, h].double() @ k[:, 0].double().T) * scale, sinks[h].double(), window or None)
            want = (p @ k[:, 0].double())[c:c + n]
            worst = max(worst, float((out[row:row + n].float().cpu().view(n, nq, d)[:, h].double() - want).abs().max()))
            top = max(top, float(want.abs().max()))
        row += n
    return worst / top


@pytest.mark.parametrize("dtype,fast", [("float32", True), ("bfloat16", True), ("bfloat16", False)])
@pytest.mark.parametrize("d,nq,page,window", [(48, 3, 4, 21), (112, 2, 8, 64), (64, 6, 16, 40), (128, 16, 16, 100), (272, 2, 8, 33),
                                              (32, 20, 4, 0)])
def test_window_and_learned_sink_in_prompt_portions(rts, dtype, fast, d, nq, page, window):
    """Portions that start before, at and behind a window's reach, beside single tokens and the first tokens of a
    sequence; for the last query of each request one key towers: the newest key its window has passed, or the oldest it
    still holds.  Sinks differ from head to head, one of them large enough to take most of the weight.  (Head sizes 64
    and 128 with pages of 8 and more: the tcgen05 kernel.)"""
    rt = rts[dtype]
    tol = 2e-5 if dtype == "float32" else 2.5e-2
    W = window or 50
    entries = [(0, 3 * W + 5), (W - 2, 7), (2 * W - 1, 1), (W + 3, 2), (5, 2 * W), (0, 2)]
    sinks = torch.linspace(-2.0, 3.0, nq)
    for which in ("outside", "inside"):
        marks = []
        for c, n in entries:
            last = c + n - 1
            oldest = max(last - W + 1, 0)
            marks.append((max(oldest - 1, 0) if which == "outside" else oldest, last))
        assert _window_sink_case(rt, entries, nq, d, page, window, sinks, seed=W, stand_out=marks, fast=fast) < tol, which


@pytest.mark.parametrize("dtype,fast", [("float32", True), ("bfloat16", True), ("bfloat16", False)])
@pytest.mark.parametrize("d,nq,page,window,splits", [(48, 3, 4, 21, None), (160, 6, 16, 40, 2), (64, 8, 8, 700, 4), (64, 8, 8, 3000, 12),
                                                     (112, 2, 8, 0, 3)])
def test_window_and_learned_sink_in_decode_steps(rts, dtype, fast, d, nq, page, window, splits):
    """Every request brings one token: at the start of a sequence, just before, at and just behind the first position whose
    window leaves a key out, deep in a long sequence (split key ranges, merged in a cluster and through scratch)."""
    rt = rts[dtype]
    tol = 2e-5 if dtype == "float32" else 2.5e-2
    W = window or 700
    entries = [(p, 1) for p in (0, 1, W - 2, W - 1, W, W + 1, 2 * W + W // 2, W // 2)]
    sinks = torch.linspace(2.5, -1.5, nq)
    for which in ("outside", "inside"):
        marks = [((max(p - W, 0) if window else 0) if which == "outside" else max(p - W + 1, 0), p) for p, _ in entries]
        assert _window_sink_case(rt, entries, nq, d, page, window, sinks, seed=W, stand_out=marks, splits=splits, fast=fast) < tol, which


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,E,top,F,shared", [(96, 5, 2, 48, True), (64, 8, 3, 16, False), (128, 4, 1, 72, False), (200, 37, 4, 40, True)])
def test_router_and_experts(rts, dtype, H, E, top, F, shared):
    """Batches of 1, 7 and 150 tokens: the choice and the weights against the plain router, the experts' weighted sum
    against the plain loop; a token's result is the same alone and in the batch (float32: to the bit)."""
    rt = rts[dtype]
    g = torch.Generator().manual_seed(E * 10 + top)
    dev = lambda t: t.to(rt.device)  # noqa: E731
    h_all = torch.randn(150, H, generator=g).to(rt.dtype)
    w_router = torch.randn(E, H, generator=g) * 0.5
    w_gu = (torch.randn(E, 2 * F, H, generator=g) / math.sqrt(H)).to(rt.dtype)
    w_dn = (torch.randn(E, H, F, generator=g) / math.sqrt(F)).to(rt.dtype)
    sh = torch.randn(150, H, generator=g).to(rt.dtype) if shared else None
    idx, wt = PT.route(h_all.double(), w_router.double(), top)
    want = torch.zeros(150, H, dtype=torch.float64)
    for t in range(150):
        for k in range(top):
            e = int(idx[t, k])
            gu = w_gu[e].double() @ h_all[t].double()
            want[t] += wt[t, k] * (w_dn[e].double() @ (PT.silu(gu[:F]) * gu[F:]))
        if shared:
            want[t] += sh[t].double()
    outs = {}
    for T in (150, 7, 1):
        entries = [(0, T)]
        ctx, _ = K.make_context(rt, entries, 4, _tables(entries, 4)[0])
        h = dev(h_all[:T])
        ids = torch.full((T, top), -1, dtype=torch.int32, device=rt.device)
        wts = torch.full((T, top), float("nan"), device=rt.device)
        rt.ops.moe_route(h, dev(w_router), ids, wts, ctx.meta)
        assert torch.equal(ids.cpu().long(), idx[:T]) and _err(wts, wt[:T]) < 1e-5
        out = torch.full((T, H), float("nan"), dtype=rt.dtype, device=rt.device)
        rt.ops.moe_experts(h, ids, wts, dev(w_gu), dev(w_dn), dev(sh[:T]) if shared else None, out, ctx.meta)
        assert _err(out, want[:T]) < (2e-5 if dtype == "float32" else 2e-2), T
        outs[T] = out.cpu()
    rt.ops.check_status()
    if dtype == "float32":
        assert torch.equal(outs[7], outs[150][:7]) and torch.equal(outs[1], outs[150][:1])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gelu(rts, dtype):
    rt = rts[dtype]
    entries = [(0, 9)]
    ctx, _ = K.make_context(rt, entries, 4, _tables(entries, 4)[0])
    for n in (64, 37):
        z = (torch.randn(9, n) * 3).to(rt.dtype)
        out = torch.empty(9, n, dtype=rt.dtype, device=rt.device)
        rt.ops.activation(z.to(rt.device), out, "gelu_tanh", ctx.meta)
        assert _err(out, PT.gelu_tanh(z.double())) < (1e-6 if dtype == "float32" else 1e-2)
