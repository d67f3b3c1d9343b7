"""The plain Dosovik against what its mechanisms must do, each alone (CPU)."""
import math

import torch

import plain_dosovik as PD


def test_short_conv_is_causal_and_starts_from_zeros():
    g = torch.Generator().manual_seed(0)
    h, w = torch.randn(9, 5, generator=g, dtype=torch.float64), torch.randn(5, 4, generator=g, dtype=torch.float64)
    y = PD.short_conv(h, w)
    assert torch.allclose(y[0], w[:, 3] * h[0])                      # only the newest tap sees the first row
    assert torch.allclose(y[3], (w * h[0:4].T).sum(1))               # all four taps, oldest first
    h2 = h.clone()
    h2[6:] += 1.0
    assert torch.equal(PD.short_conv(h2, w)[:6], y[:6])              # nothing looks ahead


def test_sink_takes_its_share_and_chunks_hide_earlier_keys():
    g = torch.Generator().manual_seed(1)
    q, k = torch.randn(7, 2, 8, generator=g, dtype=torch.float64), torch.randn(7, 1, 8, generator=g, dtype=torch.float64)
    v = torch.ones(7, 1, 3, dtype=torch.float64)
    out = PD.chunk_sink_attention(q, k, v, 0.5, chunk=3)
    # values all one: the output is the weights' sum, 1 - 1 / (1 + sum exp(s)) over the visible keys only
    for i in range(7):
        s = (k[(i // 3) * 3:i + 1, 0] @ q[i, 1]) * 0.5
        assert math.isclose(float(out[i, 1, 0]), float(torch.exp(s).sum() / (1 + torch.exp(s).sum())), rel_tol=1e-12)
    # position 3 opens a chunk: it sees itself alone, whatever the keys before it are
    k2 = k.clone()
    k2[:3] *= 50.0
    assert torch.allclose(PD.chunk_sink_attention(q, k2, v, 0.5, chunk=3)[3:], out[3:])


def test_partial_rotation_keeps_the_tail_and_depends_on_distance():
    g = torch.Generator().manual_seed(2)
    x = torch.randn(1, 1, 12, generator=g, dtype=torch.float64)
    a = PD.partial_rotation(x.expand(5, 1, 12), torch.arange(5), 8, 100.0)
    assert torch.equal(a[:, :, 8:], x[:, :, 8:].expand(5, 1, 4))
    assert torch.allclose(a[..., :8].norm(dim=-1), x[..., :8].norm(dim=-1).expand(5, 1))
    assert torch.allclose(a[0], x[0])                                # position 0: angle zero
    d1 = (a[1, 0, :8] * a[3, 0, :8]).sum()
    d2 = (a[2, 0, :8] * a[4, 0, :8]).sum()
    assert math.isclose(float(d1), float(d2), rel_tol=1e-12)          # same distance, same product


def test_poly_norm_terms():
    z = torch.tensor([[1.0, -2.0, 3.0, 0.5]], dtype=torch.float64)
    n = lambda u: u / torch.sqrt((u * u).mean() + 1e-6)              # noqa: E731
    for coef, want in (([1, 0, 0, 0], n(z)), ([0, 1, 0, 0], n(z * z)), ([0, 0, 1, 0], n(z ** 3)), ([0, 0, 0, 2.5], torch.full_like(z, 2.5))):
        assert torch.allclose(PD.poly_norm(z, torch.tensor(coef, dtype=torch.float64), 1e-6), want)


def test_one_plus_norm_with_zero_weight_is_the_plain_division():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    assert torch.allclose(PD.one_plus_norm(x, torch.zeros(2, dtype=torch.float64), 0.0), x / math.sqrt(12.5))
