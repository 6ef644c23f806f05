"""The plain Pekunex against closed forms and against itself, and the engine's configuration of the
design (no GPU needed)."""

import copy
import math

import pytest
import torch

from tests.pekunex_configs import PEK, PEK_LONG, pekunex_weights, random_ids, tensor_shapes
from tests.plain import pekunex_plain as plain


def test_sink_softmax_is_a_softmax_with_one_more_key():
    s = torch.randn(6, 6, dtype=torch.float64, generator=torch.Generator().manual_seed(1))
    w = plain.causal_weights(s, sink=0.7)
    for i in range(6):
        row = torch.cat([s[i, : i + 1], torch.tensor([0.7], dtype=torch.float64)])
        assert torch.allclose(w[i, : i + 1], torch.softmax(row, 0)[:-1], atol=1e-12)
        assert float(w[i, i + 1:].abs().sum()) == 0.0
    assert torch.allclose(plain.causal_weights(s).sum(-1), torch.ones(6, dtype=torch.float64))
    assert float(plain.causal_weights(s, sink=30.0).sum(-1).max()) < 1e-9  # a large sink takes nearly everything


def test_rotation_turns_the_first_entries_scales_them_and_keeps_the_rest():
    x = torch.randn(5, 2, 12, dtype=torch.float64, generator=torch.Generator().manual_seed(2))
    f = plain.base_frequencies(100.0, 8)
    y = plain.rotate_halves(x, [0, 1, 2, 50, 900], f, 1.25)
    assert torch.equal(y[..., 8:], x[..., 8:])
    assert torch.allclose(y[0, :, :8], 1.25 * x[0, :, :8])
    assert torch.allclose(y[..., :8].norm(dim=-1), 1.25 * x[..., :8].norm(dim=-1))
    # the angle between a query and a key depends on the distance only
    a = plain.rotate_halves(x[:1], [7], f, 1.0)[0, 0, :8] @ plain.rotate_halves(x[1:2], [3], f, 1.0)[0, 0, :8]
    b = plain.rotate_halves(x[:1], [104], f, 1.0)[0, 0, :8] @ plain.rotate_halves(x[1:2], [100], f, 1.0)[0, 0, :8]
    assert abs(float(a - b)) < 1e-9


def test_smooth_stretch_keeps_fast_waves_and_slows_long_ones():
    base, dims = 10000.0, 32
    s = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
    f, mag = plain.smooth_stretch(base, dims, s)
    f0 = plain.base_frequencies(base, dims)
    assert mag == pytest.approx(0.1 * math.log(4.0) + 1.0)
    assert float(f[0]) == float(f0[0]) and float(f[-1]) == pytest.approx(float(f0[-1]) / 4.0)
    assert bool(((f <= f0) & (f >= f0 / 4.0 - 1e-18)).all())
    ratio = f0 / f
    assert bool((ratio[1:] >= ratio[:-1] - 1e-12).all())  # the ramp only rises
    # lo and hi by hand: the pair index at which a wave makes `turns` turns over the original length
    idx = lambda turns: dims * math.log(64 / (2 * math.pi * turns)) / (2 * math.log(base))
    lo, hi = max(math.floor(idx(8.0)), 0), min(math.ceil(idx(1.0)), dims - 1)
    for i in range(dims // 2):
        r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        assert float(f[i]) == pytest.approx(float(f0[i]) * (r / 4.0 + 1.0 - r))


def test_piecewise_stretch_has_three_branches():
    base, dims = 5000.0, 32
    s = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 40}
    f, mag = plain.piecewise_stretch(base, dims, s)
    f0 = plain.base_frequencies(base, dims)
    wave = 2 * math.pi / f0
    kinds = set()
    for i in range(dims // 2):
        if wave[i] < 40 / 4.0:
            kinds.add("kept")
            assert float(f[i]) == float(f0[i])
        elif wave[i] > 40 / 1.0:
            kinds.add("slowed")
            assert float(f[i]) == pytest.approx(float(f0[i]) / 8.0)
        else:
            kinds.add("between")
            t = (40 / float(wave[i]) - 1.0) / 3.0
            assert float(f[i]) == pytest.approx((1 - t) * float(f0[i]) / 8.0 + t * float(f0[i]))
    assert kinds == {"kept", "slowed", "between"} and mag == 1.0


def test_matrix_memory_equals_the_stabilised_sum_over_earlier_tokens():
    g = torch.Generator().manual_seed(3)
    T, d, e = 9, 5, 4
    q, k, v = (torch.randn(T, n, dtype=torch.float64, generator=g) for n in (d, d, e))
    log_i = torch.randn(T, dtype=torch.float64, generator=g) * 2
    log_f = torch.nn.functional.logsigmoid(torch.randn(T, dtype=torch.float64, generator=g) + 2)
    out, (S, n, m) = plain.matrix_memory_recurrence(q, k, v, log_i, log_f)
    F = torch.cumsum(log_f, 0)
    for t in range(T):
        w = torch.tensor([float(F[t] - F[s] + log_i[s]) for s in range(t + 1)], dtype=torch.float64)
        m_t = max(float(F[t]), float(w.max()))  # the running maximum starts at 0: the first term is the decayed start
        num = sum(math.exp(float(w[s]) - m_t) * float(k[s] @ q[t]) * v[s] for s in range(t + 1))
        den = sum(math.exp(float(w[s]) - m_t) * float(k[s] @ q[t]) for s in range(t + 1))
        assert torch.allclose(out[t], num / (max(abs(den), math.exp(-m_t)) + 1e-6), atol=1e-10)
    assert m == pytest.approx(m_t)
    # cut anywhere: the state carries everything
    a, st = plain.matrix_memory_recurrence(q[:4], k[:4], v[:4], log_i[:4], log_f[:4])
    b, _ = plain.matrix_memory_recurrence(q[4:], k[4:], v[4:], log_i[4:], log_f[4:], state=st)
    assert torch.allclose(torch.cat([a, b]), out, atol=1e-12)


def test_state_space_equals_the_decayed_sum_and_convolution_keeps_its_last_inputs():
    g = torch.Generator().manual_seed(4)
    T, e, N = 8, 3, 4
    x, B, C = (torch.randn(T, n, dtype=torch.float64, generator=g) for n in (e, N, N))
    dt = torch.rand(T, dtype=torch.float64, generator=g) * 0.5
    out, S = plain.state_space_recurrence(x, B, C, dt, 1.7, 0.3)
    for t in range(T):
        want = 0.3 * x[t]
        for s in range(t + 1):
            want = want + math.exp(-1.7 * float(dt[s + 1: t + 1].sum())) * float(dt[s]) * float(B[s] @ C[t]) * x[s]
        assert torch.allclose(out[t], want, atol=1e-12)
    taps, bias = torch.randn(6, 4, dtype=torch.float64, generator=g), torch.randn(6, dtype=torch.float64, generator=g)
    u = torch.randn(T, 6, dtype=torch.float64, generator=g)
    whole = plain.short_convolution(u, taps, bias)
    assert torch.allclose(whole[0], bias + taps[:, 3] * u[0])
    for cut in (1, 2, 5):
        before = torch.cat([torch.zeros(3, 6, dtype=torch.float64), u[:cut]])[-3:]
        assert torch.allclose(plain.short_convolution(u[cut:], taps, bias, before=before), whole[cut:], atol=1e-12)


@pytest.mark.parametrize("tag", ["a", "b", "c", "e"])
def test_logits_of_a_prefix_do_not_depend_on_what_follows(tag):
    cfg = PEK[tag]
    w = pekunex_weights(cfg, 7)
    ids = random_ids(cfg, 45, 70)
    whole = plain.forward_logits(ids, w, cfg)
    assert torch.allclose(plain.forward_logits(ids[:19], w, cfg), whole[:19], atol=1e-10)


def test_a_layer_with_borrowed_weights_equals_its_own_copy_of_them():
    cfg = PEK["a"]
    w = pekunex_weights(cfg, 9)
    own = copy.deepcopy(cfg)
    w2 = dict(w)
    for i, layer in enumerate(own["layers"]):
        j = layer.pop("weights_of", None)
        if j is not None:
            w2.update({f"l{i}." + k[len(f"l{j}."):]: v for k, v in w.items() if k.startswith(f"l{j}.")})
    ids = random_ids(cfg, 30, 5)
    assert torch.equal(plain.forward_logits(ids, w, cfg), plain.forward_logits(ids, w2, own))


# ---------------------------------------------------------------------------
# the engine's configuration, registry and run order


@pytest.mark.parametrize("cfg", list(PEK.values()) + [PEK_LONG])
def test_config_and_tensor_names(cfg):
    from tokensprint_b200.config.registry import architecture_for

    arch = architecture_for(cfg)
    typed = arch.config_from_dict(cfg)
    assert typed.to_dict() == cfg
    spec = arch.build_spec(typed)
    want = tensor_shapes(cfg)
    got = {s.name: tuple(s.shape) for s in spec.tensor_specs()}
    assert set(got) | set(spec.ignorable_tensors) == set(want)
    assert all(shape == want[name] for name, shape in got.items())
    owners = [i if l.get("weights_of") is None else l["weights_of"] for i, l in enumerate(cfg["layers"])]
    own = [i for i, l in enumerate(cfg["layers"]) if l.get("weights_of") is None]
    assert [own[r.layer] for r in spec.run_order] == owners
    assert all(r.cache is None for r in spec.run_order)  # a cache and a state of its own for every run


def test_frequencies_of_the_engine_equal_the_plain_ones():
    from tokensprint_b200.parts.position import scaled_frequencies

    for base, dims, s in ((10000.0, 8, {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}),
                          (500000.0, 64, {"factor": 16.0, "original": 1000, "fast": 32.0, "slow": 0.25}),
                          (300.0, 2, {"factor": 2.0, "original": 5, "fast": 3.0, "slow": 2.0})):
        f, mag = scaled_frequencies(dims, base, dict(s, kind="yarn"))
        want, wmag = plain.smooth_stretch(base, dims, s)
        assert torch.allclose(f, want, rtol=1e-14, atol=0) and mag == pytest.approx(wmag, rel=1e-14)
    for base, dims, s in ((5000.0, 16, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 32}),
                          (1000000.0, 128, {"factor": 32.0, "low": 0.5, "high": 3.0, "original": 700})):
        f, mag = scaled_frequencies(dims, base, dict(s, kind="llama3"))
        assert torch.allclose(f, plain.piecewise_stretch(base, dims, s)[0], rtol=1e-14, atol=0) and mag == 1.0
    f, mag = scaled_frequencies(12, 77.0, None)
    assert torch.allclose(f, plain.base_frequencies(77.0, 12), rtol=1e-14, atol=0) and mag == 1.0


def test_config_errors_name_the_key():
    from tokensprint_b200.config.model_config import ConfigError
    from tokensprint_b200.models.pekunex import PekunexConfig

    cases = ((("layers", 0, "type"), "conv"), (("layers", 0, "mixer", "kv_heads"), 3), (("layers", 0, "mixer", "rot", "dims"), 7),
             (("layers", 0, "mixer", "rot", "dims"), 26), (("layers", 3, "weights_of"), 3), (("layers", 3, "weights_of"), 1),
             (("layers", 4, "weights_of"), 3), (("layers", 2, "mixer", "groups"), 3), (("layers", 2, "mixer", "norm_groups"), 5),
             (("layers", 1, "mixer", "right", "gate_cap"), 0.0), (("layers", 0, "mlp", "kind"), "moe"), (("norm", "eps"), 0.0))
    for path, value in cases:
        bad = copy.deepcopy(PEK["a"])
        node = bad
        for key in path[:-1]:
            node = node[key]
        node[path[-1]] = value
        with pytest.raises(ConfigError):
            PekunexConfig.from_dict(bad)


def test_random_weights_and_presets():
    from tokensprint_b200.config.registry import architecture_for
    from tokensprint_b200.weights.loader import RandomSource

    cfg = PEK["b"]
    arch = architecture_for(cfg)
    shapes = RandomSource(arch.build_spec(arch.config_from_dict(cfg)).tensor_specs(), 1).shapes()
    want = tensor_shapes(cfg)
    assert all(tuple(shapes[k]) == want[k] for k in shapes)


def test_cache_needs_of_the_mixers():
    """Pages for the attentions (keys and values padded to one width), a state slot for the
    recurrent mixers, both for the pair side by side."""
    from tokensprint_b200.models.model import Model
    from tokensprint_b200.models.pekunex import PekunexConfig, build_pekunex_spec

    cfg = PEK["a"]
    model = Model(build_pekunex_spec(PekunexConfig.from_dict(cfg)), torch.device("cpu"), torch.float32)
    needs = [model.blocks[r.layer].mixer.cache_need() for r in model.spec.run_order]
    assert [n.kind for n in needs] == ["full", "full", "none", "none", "full"]
    assert needs[0].k_row == (2, 24) and needs[0].state_shape is None
    assert needs[1].k_row == (1, 20) and needs[1].state_shape == (3 * 12 * 21 + 3,)
    assert needs[2].state_shape == (4 * 8 * 12 + 2 * (48 + 2 * 16),)


def test_long_portions_run_in_segments_only_while_the_grid_is_small():
    from tokensprint_b200 import ops

    few = ops.gla_ctas_per_sequence(4, 32, 49)      # 4 heads, a block of 64 columns each
    many = ops.gla_ctas_per_sequence(128, 128, 64)  # 128 heads, four blocks of 16 columns each
    assert few == 4 and many == 512
    assert ops.gla_segments(1, 1200, few) == (5, 256) and ops.gla_segments(1, 300, few) == (1, 0)
    assert ops.gla_segments(1, 1200, many) == (1, 0) and ops.gla_segments(80, 1200, few) == (1, 0)
    assert ops.gla_segments(1, 1200) == (5, 256) and ops.gla_segments(1, None, few) == (1, 0)
