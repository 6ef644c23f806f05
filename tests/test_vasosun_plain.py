"""Host tests of Vasosun: the plain model's mechanisms against independent restatements and against
properties the design implies, and the engine's configuration and specification (no GPU)."""

import math

import pytest
import torch

from tests.plain import vasosun_plain as plain
from tests.vasosun_configs import VAS, VAS_LONG, random_ids, tensor_shapes, vasosun_weights


def _w(cfg, seed=5, **kw):
    return {k: v.double() for k, v in vasosun_weights(cfg, seed, **kw).items()}


def test_convolution_against_explicit_sums():
    g = torch.Generator().manual_seed(1)
    for taps in (1, 2, 3, 5):
        h, w = torch.randn(9, 4, generator=g, dtype=torch.float64), torch.randn(4, taps, generator=g, dtype=torch.float64)
        want = torch.zeros_like(h)
        for t in range(9):
            for j in range(taps):
                src = t - taps + 1 + j
                if src >= 0:
                    want[t] += w[:, j] * h[src]
        assert torch.allclose(plain.causal_conv(h, w), want, atol=1e-12)
        # the last tap weighs the current token
        assert torch.allclose(plain.causal_conv(h, w)[0], w[:, -1] * h[0], atol=1e-12)


def test_pair_rows():
    assert plain.pair_rows([5, 9, 2], 97, 7, 13) == [97, (5 * 7 + 9 * 13) % 97, (9 * 7 + 2 * 13) % 97]
    assert plain.pair_rows([3], 10, 1, 1) == [10]


def test_delta_rule_against_the_transition_form_and_overwriting():
    g = torch.Generator().manual_seed(2)
    T, d, e = 12, 5, 3
    q, k, v = (torch.randn(T, n, generator=g, dtype=torch.float64) for n in (d, d, e))
    k = k / k.norm(dim=-1, keepdim=True)
    decay, beta = torch.rand(T, generator=g, dtype=torch.float64), torch.rand(T, generator=g, dtype=torch.float64)
    got = plain.delta_recurrence(q, k, v, decay, beta)
    S = torch.zeros(d, e, dtype=torch.float64)
    for t in range(T):  # S_t = (I - beta k k^T) g S_(t-1) + beta k v^T
        S = (torch.eye(d, dtype=torch.float64) - beta[t] * torch.outer(k[t], k[t])) @ (decay[t] * S) + beta[t] * torch.outer(k[t], v[t])
        assert torch.allclose(got[t], S.T @ q[t], atol=1e-12)
    # with full write strength and a unit key, what was written for a key is read back as it was written
    one = plain.delta_recurrence(k[:1], k[:1], v[:1], torch.ones(1, dtype=torch.float64), torch.ones(1, dtype=torch.float64))
    assert torch.allclose(one[0], v[0], atol=1e-12)
    again = plain.delta_recurrence(k[[0, 0]], k[[0, 0]], torch.stack([v[0], v[1]]), torch.ones(2, dtype=torch.float64), torch.ones(2, dtype=torch.float64))
    assert torch.allclose(again[1], v[1], atol=1e-12)  # the second write replaces the first


def test_window_edges_and_distance_penalty():
    cfg = VAS["a"]
    W = _w(cfg, sharp=3.0)
    m, p = cfg["layers"][0]["mixer"], "l0.mix."
    size = m["mask"]["size"]
    g = torch.Generator().manual_seed(3)
    h = torch.randn(size + 6, cfg["width"], generator=g, dtype=torch.float64)
    pos = list(range(h.shape[0]))
    base = plain.window_attention(h, pos, m, W, p)
    i = size + 2
    outside, inside = i - size, i - size + 1
    for j, seen in ((outside, False), (inside, True)):
        h2 = h.clone()
        h2[j] += 1.0
        moved = (plain.window_attention(h2, pos, m, W, p)[i] - base[i]).abs().max()
        assert (moved > 1e-6) == seen
    # the penalty alone: equal keys and values everywhere, so a head's weights follow -r1 ln(1 + r2 distance)
    T = 9
    r1, r2 = W[p + "r1"], W[p + "r2"]
    scores = -r1[0] * torch.log1p(r2[0] * torch.arange(T - 1, -1, -1, dtype=torch.float64))
    assert torch.allclose(plain.softmax_over_visible(scores[None, :], torch.ones(1, T, dtype=torch.bool))[0].log().diff(),
                          scores.diff(), atol=1e-12)
    t = plain.query_temperature([0, 6, 7, 8, 15, 16], 0.7, 8)
    assert torch.allclose(t, torch.tensor([1.0, 1.0, 1 + 0.7 * math.log(2), 1 + 0.7 * math.log(2), 1 + 0.7 * math.log(3), 1 + 0.7 * math.log(3)], dtype=torch.float64))


def test_stretched_frequencies_and_neighbour_rotation():
    f, mag = plain.stretched_frequencies(1000.0, 6, {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0})
    base = [1000.0 ** (-2 * i / 6) for i in range(3)]
    index = lambda turns: 6 * math.log(32 / (2 * math.pi * turns)) / (2 * math.log(1000.0))
    lo, hi = max(math.floor(index(8.0)), 0), min(math.ceil(index(1.0)), 5)
    for i in range(3):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        assert abs(float(f[i]) - (base[i] / 4.0 * ramp + base[i] * (1 - ramp))) < 1e-15
    assert abs(mag - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    x = torch.arange(1.0, 9.0, dtype=torch.float64).view(1, 1, 8)
    y = plain.rotate_neighbours(x, [3], torch.tensor([0.5], dtype=torch.float64), 2.0)
    c, s = 2.0 * math.cos(1.5), 2.0 * math.sin(1.5)
    assert torch.allclose(y[0, 0, :2], torch.tensor([1 * c - 2 * s, 2 * c + 1 * s], dtype=torch.float64))
    assert torch.equal(y[0, 0, 2:], x[0, 0, 2:])  # entries behind the rotated ones stay


def test_latent_attention_equals_its_absorbed_form():
    """Scores against the latent through U_k^T q, values through U_v on the weighted latent: what an engine may compute instead."""
    cfg = VAS["a"]
    W = _w(cfg)
    m, p, eps = cfg["layers"][1]["mixer"], "l1.mix.", cfg["norm"]["eps"]
    g = torch.Generator().manual_seed(4)
    T = 11
    h = torch.randn(T, cfg["width"], generator=g, dtype=torch.float64)
    pos = list(range(T))
    c, kr = plain.latent_rows(h, pos, m, W, p, eps)
    want = plain.latent_attention(h, pos, m, W, p, eps, c, kr)
    H, d, r, e, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = plain.unit_rms(h @ W[p + "dq"].T, eps) * W[p + "dq.norm"]
    q = (cq @ W[p + "uq"].T).view(T, H, d + r)
    f, mag = plain.stretched_frequencies(m["rot"]["base"], m["rot"]["dims"], m["rot"].get("scaling"))
    qr = plain.rotate_neighbours(q[..., d:], pos, f, mag)
    uk, uv = W[p + "uk"].view(H, d, R), W[p + "uv"].view(H, e, R)
    heads = []
    for a in range(H):
        s = ((q[:, a, :d] @ uk[a]) @ c.T + qr[:, a] @ kr.T) * m["scale"]
        wts = torch.softmax(s.masked_fill(~torch.ones(T, T, dtype=torch.bool).tril(), float("-inf")), -1)
        heads.append((wts @ c) @ uv[a].T)
    assert torch.allclose(torch.cat(heads, -1) @ W[p + "o"].T, want, atol=1e-10)


def test_routing_identity_experts_and_correction():
    cfg = VAS["a"]
    W = _w(cfg)
    mlp, p = cfg["layers"][1]["mlp"], "l1.mlp."
    E = mlp["router"]["experts"]
    g = torch.Generator().manual_seed(6)
    h = torch.randn(40, cfg["width"], generator=g, dtype=torch.float64)
    chosen, weights = plain.route(h, mlp, W, p)
    scores = torch.softmax(h @ W[p + "router"].T, -1)
    assert torch.allclose(weights, torch.gather(scores, 1, chosen)) and bool((weights.sum(-1) < 1).all())  # the scores themselves, not renormalised
    assert bool((chosen >= E).any()), "the test wants some identity choices"
    # a large correction on one expert makes every token choose it, and leaves its weight alone
    W2 = dict(W)
    W2[p + "correction"] = W[p + "correction"].clone()
    W2[p + "correction"][2] += 10.0
    chosen2, weights2 = plain.route(h, mlp, W2, p)
    assert bool((chosen2 == 2).any(-1).all()) and torch.allclose(weights2[chosen2 == 2], scores[:, 2])
    # an identity expert returns its input times the weight
    only = torch.full((40, 1), E, dtype=torch.long)
    out = plain.routed_ff(h, mlp, W, p, chosen=only, weights=torch.full((40, 1), 0.25, dtype=torch.float64))
    assert torch.allclose(out, 0.25 * h)
    # an expert is W_down gelu(W_up h) with the exact gelu
    one = plain.routed_ff(h[:1], mlp, W, p, chosen=torch.tensor([[1]]), weights=torch.ones(1, 1, dtype=torch.float64))
    z = h[0] @ W[p + "e1.up"].T
    assert torch.allclose(one[0], (0.5 * z * (1 + torch.erf(z / math.sqrt(2)))) @ W[p + "e1.down"].T)


@pytest.mark.parametrize("tag", sorted(VAS))
def test_a_prefix_gives_the_same_logits(tag):
    """Nothing looks ahead: convolutions, windows, recurrences and the pair table see earlier tokens only."""
    cfg = VAS[tag]
    W = _w(cfg)
    ids = random_ids(cfg, 40, 9)
    whole = plain.forward_logits(ids, W, cfg)
    part = plain.forward_logits(ids[:23], W, cfg)
    assert torch.allclose(whole[:23], part, atol=1e-9)
    assert float(whole.abs().max()) < cfg["logit_softcap"]
    assert len(plain.forward_stream(ids, W, cfg)) == len(cfg["layers"]) + 1


@pytest.mark.parametrize("cfg", list(VAS.values()) + [VAS_LONG])
def test_the_engine_reads_the_configuration_and_wants_the_same_tensors(cfg):
    from tokensprint_b200.config.registry import ARCHITECTURES
    import tokensprint_b200.models  # noqa: F401

    arch = ARCHITECTURES["Vasosun"]
    config = arch.config_from_dict(cfg)
    assert config.to_dict() == cfg
    spec = arch.build_spec(config)
    assert {s.name: tuple(s.shape) for s in spec.tensor_specs()} == tensor_shapes(cfg)
    readers = [i for i, l in enumerate(cfg["layers"]) if l["mixer"].get("kv_from") is not None]
    for i in readers:
        run = spec.run_order[i]
        assert run.cache == cfg["layers"][i]["mixer"]["kv_from"] and not run.writes_cache


def test_configurations_the_engine_refuses():
    from tokensprint_b200.config.model_config import ConfigError
    from tokensprint_b200.models.vasosun import VasosunConfig
    import copy

    bad = copy.deepcopy(VAS["a"])
    bad["layers"][3]["mixer"]["kv_from"] = 2  # a delta layer caches no latent rows
    with pytest.raises(ConfigError):
        VasosunConfig.from_dict(bad)
    bad = copy.deepcopy(VAS["a"])
    bad["layers"][3]["mixer"]["kv_rank"] = 24  # another latent width than its source's
    with pytest.raises(ConfigError):
        VasosunConfig.from_dict(bad)
    bad = copy.deepcopy(VAS["a"])
    bad["layers"][1]["mlp"]["router"]["top"] = 8  # more choices than router outputs
    with pytest.raises(ConfigError):
        VasosunConfig.from_dict(bad)
    bad = copy.deepcopy(VAS["b"])
    bad["layers"][0]["type"] = "mamba2"
    with pytest.raises(ConfigError):
        VasosunConfig.from_dict(bad)
