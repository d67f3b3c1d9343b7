"""The plain Tutezen implementation against what each mechanism must do, without the engine."""
import math

import torch

import plain_tutezen as PT

torch.manual_seed(0)
F64 = torch.float64


def test_convolution_is_causal_starts_from_zeros_and_ends_on_the_current_token():
    u, w, b = torch.randn(9, 5, dtype=F64), torch.randn(5, 3, dtype=F64), torch.randn(5, dtype=F64)
    y = PT.causal_conv(u, w, b)
    assert torch.allclose(y[0], b + w[:, 2] * u[0])                                   # the last column is the current token's
    assert torch.allclose(y[4], b + w[:, 0] * u[2] + w[:, 1] * u[3] + w[:, 2] * u[4])
    u2 = u.clone()
    u2[6:] += 1.0
    assert torch.equal(PT.causal_conv(u2, w, b)[:6], y[:6])                           # later rows change nothing earlier


def test_recurrence_equals_its_unrolled_sum_and_uses_the_heads_group():
    T, H, P, N, G = 7, 4, 3, 5, 2
    x, B, C = torch.randn(T, H, P, dtype=F64), torch.randn(T, G, N, dtype=F64), torch.randn(T, G, N, dtype=F64)
    dt, a_log, d = torch.rand(T, H, dtype=F64) + 0.1, torch.randn(H, dtype=F64), torch.randn(H, dtype=F64)
    y = PT.state_space(x, B, C, dt, a_log, d, G)
    for h in (0, 3):
        g = h // (H // G)
        t = T - 1
        want = d[h] * x[t, h]
        for s in range(t + 1):  # y_t = sum_s (C_t . B_s) exp(-rate * sum_{s < r <= t} dt_r) dt_s x_s
            decay = torch.exp(-torch.exp(a_log[h]) * dt[s + 1:t + 1, h].sum())
            want = want + (C[t, g] @ B[s, g]) * decay * dt[s, h] * x[s, h]
        assert torch.allclose(y[t, h], want)
    B2 = B.clone()
    B2[:, 1] += 1.0                                                                    # the second group's B
    y2 = PT.state_space(x, B2, C, dt, a_log, d, G)
    assert torch.equal(y2[:, :2], y[:, :2]) and not torch.allclose(y2[:, 2:], y[:, 2:])


def test_gate_comes_before_the_norm_and_parts_are_normed_alone():
    v = torch.randn(3, 12, dtype=F64)
    out = PT.grouped_rms(v, 3, 0.0)
    assert torch.allclose((out.reshape(3, 3, 4) ** 2).mean(-1), torch.ones(3, 3, dtype=F64))
    v2 = v.clone()
    v2[:, 4:8] *= 5.0                                                                  # one part scaled: the others do not move
    out2 = PT.grouped_rms(v2, 3, 0.0)
    assert torch.allclose(out2[:, :4], out[:, :4]) and torch.allclose(out2[:, 4:8], out[:, 4:8])


def test_rotation_pairs_neighbours_keeps_the_tail_and_depends_on_distance():
    q, k = torch.randn(1, 10, dtype=F64), torch.randn(1, 10, dtype=F64)
    r = PT.rotate_pairs(q, torch.tensor([3]), 6, 100.0)
    assert torch.equal(r[:, 6:], q[:, 6:])
    a = 3 * 100.0 ** (-2.0 / 6)                                                        # pair i = 1: dimensions 2 and 3
    assert torch.allclose(r[0, 2], q[0, 2] * math.cos(a) - q[0, 3] * math.sin(a))
    assert torch.allclose(r[0, 3], q[0, 3] * math.cos(a) + q[0, 2] * math.sin(a))
    dot = lambda pq, pk: float((PT.rotate_pairs(q, torch.tensor([pq]), 10, 1e4) * PT.rotate_pairs(k, torch.tensor([pk]), 10, 1e4)).sum())  # noqa: E731
    assert abs(dot(9, 4) - dot(105, 100)) < 1e-9


def test_window_edge_and_the_sinks_share():
    T, window = 12, 5
    s = torch.zeros(T, T, dtype=F64)
    p = PT.windowed_sink_softmax(s, torch.tensor(0.0, dtype=F64), window)
    assert torch.allclose(p[8, 4:9], torch.full((5,), 1 / 6, dtype=F64)) and float(p[8, :4].abs().sum()) == 0.0  # i - j < 5
    assert float(p[8, 9:].abs().sum()) == 0.0
    assert torch.allclose(p[1, :2], torch.full((2,), 1 / 3, dtype=F64))                # the first tokens: fewer keys, same sink
    big = PT.windowed_sink_softmax(s, torch.tensor(math.log(4.0), dtype=F64), window)  # exp(sink) = 4, unscaled, counted once
    assert torch.allclose(big[8, 4:9], torch.full((5,), 1 / 9, dtype=F64))
    full = PT.windowed_sink_softmax(s, torch.tensor(-1e9, dtype=F64), None)
    assert torch.allclose(full[8, :9].sum(), torch.tensor(1.0, dtype=F64))


def test_router_weights_and_choice():
    h, w = torch.randn(6, 8, dtype=F64), torch.randn(5, 8, dtype=F64)
    idx, wt = PT.route(h, w, 2)
    s = torch.softmax(h @ w.T, -1)
    for t in range(6):
        order = torch.argsort(s[t], descending=True)[:2]
        assert set(idx[t].tolist()) == set(order.tolist())
        assert torch.allclose(wt[t].sum(), torch.tensor(1.0, dtype=F64))
        assert torch.allclose(wt[t, 0] / wt[t, 1], s[t, idx[t, 0]] / s[t, idx[t, 1]])
    _, one = PT.route(h, w, 1)
    assert torch.allclose(one, torch.ones(6, 1, dtype=F64))                            # a single choice weighs 1


def test_gelu_is_the_tanh_form():
    z = torch.tensor([-3.0, -0.5, 0.0, 0.7, 4.0], dtype=F64)
    want = [0.5 * v * (1 + math.tanh(math.sqrt(2 / math.pi) * (v + 0.044715 * v ** 3))) for v in z.tolist()]
    assert torch.allclose(PT.gelu_tanh(z), torch.tensor(want, dtype=F64))


def test_layer_order_repeats_a_stretch_and_marks_each_pass():
    cfg = {"layers": [0] * 5, "loop": {"start": 1, "stop": 3, "times": 3}}
    assert [(i, t) for i, t, _ in PT.layer_order(cfg)] == [(0, None), (1, 0), (2, 0), (1, 1), (2, 1), (1, 2), (2, 2), (3, None), (4, None)]
    assert [first for _, _, first in PT.layer_order(cfg)] == [False, True, False, True, False, True, False, False, False]
    assert [i for i, _, _ in PT.layer_order({"layers": [0] * 3})] == [0, 1, 2]
