"""The mechanisms of Pekunex one at a time: each mixer part (and the kernels under it) against the
plain function of the same mechanism, whole prompts, portions down to one token, batches of unequal
sequences with slots and pages in any order; inputs made so that a far key, a sink or a window of
kept inputs that is one token off shows far beyond rounding."""

import math

import pytest
import torch

from tests.pekunex_configs import PEK, PEK_LONG, pekunex_weights
from tests.plain import pekunex_plain as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 3e-5, torch.bfloat16: 3e-2}


def _dev(t, dtype=None):
    return t.to("cuda", dtype) if dtype is not None else t.to("cuda")


def _i32(values):
    return torch.tensor(list(values), dtype=torch.int32, device="cuda")


def _rel(got, want) -> float:
    got, want = got.detach().double().cpu(), want.double()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))


def _mixer(cfg, layer, dtype, seed=17, sharp=2.0):
    """The mixer part of one layer, built from the engine's own specification, with the tests' weights."""
    from tokensprint_b200.models.pekunex import PekunexConfig, build_pekunex_spec
    from tokensprint_b200.parts.base import BuildContext, build_part

    W = pekunex_weights(cfg, seed, sharp=sharp)
    spec = build_pekunex_spec(PekunexConfig.from_dict(cfg)).layers[layer].params["mixer"]
    mixer = build_part("mixer", spec, BuildContext(torch.device("cuda"), dtype))
    mixer.load({s.name: _dev(W[s.name], torch.float32 if s.role == "vector" else dtype) for s in mixer.tensor_specs()})
    return mixer, {k: v.double() for k, v in W.items()}


class Harness:
    """Pages and state slots for one mixer, and steps of (sequence, its next n tokens) in any batch."""

    def __init__(self, mixer, dtype, page=16, num_pages=64, slots=5, seed=0):
        self.mixer, self.dtype, self.page = mixer, dtype, page
        need = mixer.cache_need()
        self.need = need
        self.k = self.v = self.state = None
        if need.kind != "none":
            self.k = torch.full((num_pages, page, *need.k_row), float("nan"), device="cuda", dtype=dtype)
            self.v = torch.full((num_pages, page, *need.v_row), float("nan"), device="cuda", dtype=dtype)
        if need.state_shape is not None:
            self.state = torch.zeros((slots, *need.state_shape), device="cuda", dtype=torch.float32)
        order = torch.randperm(num_pages, generator=torch.Generator().manual_seed(seed)).tolist()
        self.free_pages = order
        self.pages: dict[str, list[int]] = {}
        self.done: dict[str, int] = {}
        self.slot: dict[str, int] = {}
        self.free_slots = list(range(slots))[::-1]

    def end(self, name):
        self.free_pages = self.pages.pop(name, []) + self.free_pages  # used again first
        slot = self.slot.pop(name)
        self.free_slots.append(slot)
        del self.done[name]

    def step(self, x_by_seq: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
        from tokensprint_b200.parts.base import GroupTables, LayerCache, StepContext

        names = sorted(x_by_seq, key=lambda n: (x_by_seq[n].shape[0] != 1, n))  # single tokens first, as the runner orders them
        pos, seq, cu, ctx, slots, slot_map, rows = [], [], [0], [], [], [], []
        for b, name in enumerate(names):
            n = x_by_seq[name].shape[0]
            if name not in self.done:
                self.done[name], self.pages[name] = 0, []
                self.slot[name] = self.free_slots.pop()
                if self.state is not None:
                    self.state[self.slot[name]].zero_()
            start = self.done[name]
            while len(self.pages[name]) * self.page < start + n:
                self.pages[name].append(self.free_pages.pop(0))
            pos += range(start, start + n)
            seq += [b] * n
            cu.append(cu[-1] + n)
            ctx.append(start + n)
            slots.append(self.slot[name])
            slot_map += [self.pages[name][p // self.page] * self.page + p % self.page for p in range(start, start + n)]
            rows.append(x_by_seq[name])
            self.done[name] = start + n
        width = max(len(self.pages[n]) for n in names)
        table = [self.pages[n] + [-1] * (width - len(self.pages[n])) for n in names]
        T = cu[-1]
        lens = [x_by_seq[n].shape[0] for n in names]
        step = StepContext(num_tokens=T, num_seqs=len(names), token_ids=_i32([0] * T), positions=_i32(pos), seq_index=_i32(seq),
                           cu_seqlens_q=_i32(cu), context_lens=_i32(ctx), state_slots=_i32(slots),
                           groups=[GroupTables(_i32(sum(table, [])).view(len(names), width), _i32(slot_map))], page_size=self.page,
                           max_seqlen_q=max(lens), max_context_len=max(ctx), decode_only=all(n == 1 for n in lens),
                           decode_seqs=sum(1 for n in lens if n == 1))
        cache = LayerCache(group=0 if self.k is not None else -1, k_pages=self.k, v_pages=self.v, state=self.state, writes=True)
        out = self.mixer.forward(_dev(torch.cat(rows).to(self.dtype)), step, cache)
        from tokensprint_b200 import ops

        ops.flush_gemm_chain()
        return {name: out[cu[b]:cu[b + 1]].float().cpu() for b, name in enumerate(names)}


def _inputs(T, width, seed, dtype):
    x = torch.randn(T, width, generator=torch.Generator().manual_seed(seed))
    return x.to(dtype).float()  # what both sides read


def _in_portions(h: Harness, name, x, sizes):
    out, pos, i = [], 0, 0
    while pos < x.shape[0]:
        n = min(sizes[i % len(sizes)], x.shape[0] - pos)
        out.append(h.step({name: x[pos:pos + n]})[name])
        pos, i = pos + n, i + 1
    return torch.cat(out)


# (configuration, layer, the plain function of its mixer)
def _plain_of(cfg, layer):
    entry = cfg["layers"][layer]
    eps = cfg["norm"]["eps"]
    p = f"l{layer}.mix."
    if entry["type"] == "attention":
        return lambda x, W: plain.capped_attention(x, list(range(x.shape[0])), entry["mixer"], p, W, eps)
    if entry["type"] == "parallel":
        return lambda x, W: plain.side_by_side(x, list(range(x.shape[0])), entry["mixer"], p, W, eps)
    return lambda x, W: plain.state_space(x, entry["mixer"], p, W, eps)


MIXERS = [("a", 0), ("a", 1), ("a", 2), ("b", 0), ("b", 1), ("b", 2), ("b", 3), ("c", 0), ("c", 1), ("c", 2), ("d", 0), ("d", 1), ("d", 2), ("d", 3)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tag, layer", MIXERS)
def test_mixer_whole_in_portions_and_token_by_token(dtype, tag, layer):
    """One sequence of 77 tokens: whole; in portions of changing size (one and two tokens among them,
    shorter than the convolution's taps); token by token; all against the plain mixer."""
    cfg = PEK[tag]
    mixer, W = _mixer(cfg, layer, dtype)
    x = _inputs(77, cfg["width"], 5, dtype)
    want = _plain_of(cfg, layer)(x.double(), W)
    for what, sizes, page in (("whole", (77,), 16), ("portions", (5, 1, 2, 17, 1, 1, 3, 31, 2), 8), ("token by token", (1,), 16)):
        got = _in_portions(Harness(mixer, dtype, page=page, seed=layer), "s", x, sizes)
        assert _rel(got, want) < TOL[dtype], f"{what}: {_rel(got, want):.3g}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tag, layer", [("a", 0), ("a", 1), ("a", 2), ("b", 2), ("b", 3), ("d", 1)])
def test_mixer_batches_of_unequal_sequences_with_slots_and_pages_used_again(dtype, tag, layer):
    """Three sequences side by side (portions of one beside single tokens of another), one of them
    ends, and a fourth takes its slot and pages: every sequence equals itself alone."""
    cfg = PEK[tag]
    mixer, W = _mixer(cfg, layer, dtype)
    fn = _plain_of(cfg, layer)
    xs = {n: _inputs(T, cfg["width"], 10 + i, dtype) for i, (n, T) in enumerate((("p", 40), ("q", 9), ("r", 23), ("s", 30)))}
    want = {n: fn(x.double(), W) for n, x in xs.items()}
    h = Harness(mixer, dtype, page=8, num_pages=14, slots=3)
    got = {n: [] for n in xs}
    plan = [{"p": 20, "q": 1, "r": 3}, {"p": 1, "q": 1, "r": 20}, {"p": 2, "q": 7}, {"p": 1}, {"p": 16, "s": 1}, {"s": 29}]
    for sizes in plan:
        batch = {n: xs[n][h.done.get(n, 0):h.done.get(n, 0) + k] for n, k in sizes.items()}
        for n, o in h.step(batch).items():
            got[n].append(o)
        for n in list(h.done):
            if h.done[n] == xs[n].shape[0]:
                h.end(n)
    for n in xs:
        assert _rel(torch.cat(got[n]), want[n]) < TOL[dtype], f"sequence {n}: {_rel(torch.cat(got[n]), want[n]):.3g}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_keeps_memories_in_range(dtype):
    """600 tokens one by one through the side-by-side mixer and the state-space mixer: running maxima,
    normalisers and states stay finite and right."""
    cfg = PEK_LONG
    for layer in (1, 2):
        mixer, W = _mixer(cfg, layer, dtype, sharp=1.0)
        x = _inputs(600, cfg["width"], 3, dtype)
        want = _plain_of(cfg, layer)(x.double(), W)
        h = Harness(mixer, dtype, page=16)
        got = torch.cat([h.step({"s": x[:300]})["s"]] + [h.step({"s": x[t:t + 1]})["s"] for t in range(300, 600)])
        assert bool(torch.isfinite(got).all()) and _rel(got, want) < TOL[dtype]


# ---------------------------------------------------------------------------
# attention: inputs that make one key, the sink or the cap decide


def _paged(rows, page, dtype, seed):
    """rows [N, heads, d] into a pool whose pages are in a random order; returns (pool, table)."""
    N = rows.shape[0]
    n_pages = -(-N // page)
    order = torch.randperm(n_pages + 3, generator=torch.Generator().manual_seed(seed))[:n_pages]
    pool = torch.full((n_pages + 3, page, *rows.shape[1:]), float("nan"), dtype=dtype)
    for j in range(N):
        pool[order[j // page], j % page] = rows[j].to(dtype)
    return _dev(pool), order.to(torch.int32)


def _attend(q, k, v, q_pos, page, nq, nkv, d, scale, softcap, sinks, dtype, seed=0, kernel="simple", splits=1):
    """One sequence: keys 0..N-1 in the cache, queries at `q_pos`.  "simple": the CUDA-core kernel, any
    positions; "mma" and "tcgen05" (bfloat16): the tensor-core kernels, whose queries are the last
    len(q_pos) positions of a sequence of q_pos[-1] + 1 tokens; `splits` > 1: the keys over several CTAs."""
    from tokensprint_b200 import ops

    kp, table = _paged(k, page, dtype, seed)
    vp, _ = _paged(v, page, dtype, seed)
    T = len(q_pos)
    out = torch.empty((T, nq * d), device="cuda", dtype=dtype)
    qd, hs = _dev(q.reshape(T, nq * d).to(dtype)), None if sinks is None else _dev(sinks.float())
    if kernel == "simple":
        ops.attention_paged_simple(qd, kp, vp, out, _i32(q_pos), _i32([0] * T), _dev(table).view(1, -1), page, nq, nkv, d, scale,
                                   softcap=softcap, head_sinks=hs)
    else:
        assert list(q_pos) == list(range(q_pos[-1] + 1 - T, q_pos[-1] + 1))
        cu, lens = _i32([0, T]), _i32([q_pos[-1] + 1])
        if kernel == "tcgen05":
            ops.attention_prefill_tcgen05(qd, kp, vp, out, cu, lens, _dev(table).view(1, -1), page, 1, T, nq, nkv, scale, 0, softcap=softcap,
                                          head_sinks=hs)
        else:
            scratch = torch.empty(ops.attention_scratch_floats(T * nq, splits, d), device="cuda", dtype=torch.float32) if splits > 1 else None
            ops.attention_paged_mma(qd, kp, vp, out, cu, lens, _dev(table).view(1, -1), _i32([0] * T), page, 1, T, nq, nkv, d, scale, 0, splits,
                                    scratch, 0, softcap=softcap, head_sinks=hs)
        ops.check_device_errors()
    return out.float().cpu().reshape(T, nq, d)


def _plain_attend(q, k, v, q_pos, nq, nkv, scale, softcap, sinks):
    out = torch.empty(len(q_pos), nq, v.shape[-1], dtype=torch.float64)
    for h in range(nq):
        g = h // (nq // nkv)
        for i, p in enumerate(q_pos):
            s = (k[: p + 1, g].double() @ q[i, h].double()) * scale
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            if sinks is not None:
                s = torch.cat([s, sinks[h:h + 1].double()])
            w = torch.softmax(s, 0)[: p + 1]
            out[i, h] = w @ v[: p + 1, g].double()
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq, nkv, d, page, softcap, with_sinks", [(4, 2, 24, 8, 7.0, False), (3, 1, 16, 16, 0.0, True), (6, 6, 64, 32, 15.0, True),
                                                                   (2, 1, 128, 16, 30.0, False), (5, 5, 20, 64, 0.0, True)])
def test_capped_scores_and_sinks_random(dtype, nq, nkv, d, page, softcap, with_sinks):
    g = torch.Generator().manual_seed(nq * d)
    N = 150
    q, k, v = (torch.randn(N, h, d, generator=g).to(dtype).float() for h in (nq, nkv, nkv))
    sinks = torch.randn(nq, generator=g) * 2 if with_sinks else None
    q_pos = [0, 1, 7, 8, 63, 64, 100, 149]
    got = _attend(q[q_pos], k, v, q_pos, page, nq, nkv, d, 1.5 / math.sqrt(d), softcap, sinks, dtype)
    want = _plain_attend(q[q_pos], k, v, q_pos, nq, nkv, 1.5 / math.sqrt(d), softcap, sinks)
    assert _rel(got, want) < TOL[dtype]


@pytest.mark.parametrize("nq, nkv, d, page, softcap, with_sinks", [(4, 2, 32, 8, 7.0, False), (3, 1, 16, 16, 0.0, True), (6, 6, 64, 32, 15.0, True),
                                                                   (2, 1, 128, 16, 30.0, False), (8, 2, 128, 64, 0.0, True), (4, 4, 128, 16, 10.0, True),
                                                                   (5, 5, 48, 64, 4.0, True), (16, 2, 64, 16, 25.0, True)])
def test_capped_scores_and_sinks_on_tensor_cores(nq, nkv, d, page, softcap, with_sinks):
    """The tensor-core kernels (bfloat16): a prompt portion behind a kept prefix (the prompt kernels: mma, and
    tcgen05 at heads of 128), and single decoded tokens with the keys over 1 to 8 CTAs (the sink is
    counted once, the cap applies in every range), against the plain softmax."""
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(nq * d + 1)
    N = 333
    q, k, v = (torch.randn(N, h, d, generator=g).to(dtype).float() for h in (nq, nkv, nkv))
    sinks = torch.randn(nq, generator=g) * 2 if with_sinks else None
    scale = 1.5 / math.sqrt(d)
    want = _plain_attend(q, k, v, list(range(N)), nq, nkv, scale, softcap, sinks)
    kernels = ["mma"] + (["tcgen05"] if d == 128 and page >= 8 and (64 % page == 0 or page % 128 == 0) else [])
    for kernel in kernels:
        for first in (0, 100, 331):  # whole; behind a prefix; the last two tokens
            q_pos = list(range(first, N))
            got = _attend(q[first:], k, v, q_pos, page, nq, nkv, d, scale, softcap, sinks, dtype, kernel=kernel)
            assert _rel(got, want[first:]) < TOL[dtype], f"{kernel}, queries from {first}: {_rel(got, want[first:]):.3g}"
    for n in (1, 40, 333):
        for splits in (1, 2, 5, 8):
            got = _attend(q[n - 1:n], k[:n], v[:n], [n - 1], page, nq, nkv, d, scale, softcap, sinks, dtype, kernel="mma", splits=splits)
            assert _rel(got, want[n - 1:n]) < TOL[dtype], f"decode at {n} keys, {splits} splits: {_rel(got, want[n - 1:n]):.3g}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_far_key_among_hundreds_and_the_first_key(dtype):
    """A query that matches one key hundreds of positions back (at a page's last slot, at a page's
    first slot, at position 0) returns that key's value; under a cap the match is bent but still decides."""
    nq, nkv, d, page, N = 2, 1, 32, 16, 700
    g = torch.Generator().manual_seed(9)
    k, v = torch.randn(N, nkv, d, generator=g) * 0.1, torch.randn(N, nkv, d, generator=g)
    for far in (0, 15, 16, 351, 698):
        kk = k.clone()
        kk[far, 0] = 0
        kk[far, 0, 3] = 6.0
        q = torch.zeros(1, nq, d)
        q[0, :, 3] = 6.0
        for softcap in (0.0, 20.0):
            want = _plain_attend(q, kk.to(dtype).float(), v.to(dtype).float(), [N - 1], nq, nkv, 1.0, softcap, None)
            for kernel, splits in [("simple", 1)] + ([("mma", 1), ("mma", 4)] if dtype == torch.bfloat16 else []):
                got = _attend(q, kk.to(dtype).float(), v.to(dtype).float(), [N - 1], page, nq, nkv, d, 1.0, softcap, None, dtype, seed=far,
                              kernel=kernel, splits=splits)
                assert _rel(got, want) < TOL[dtype]
                assert float((got[0, 0] - v[far, 0].to(dtype).float()).abs().max()) < 0.05, f"key {far} was not found (cap {softcap}, {kernel})"


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_cap_bounds_a_large_score_and_a_sink_takes_its_share(dtype):
    nq, nkv, d, page, N = 2, 2, 16, 8, 40
    g = torch.Generator().manual_seed(4)
    k, v = torch.randn(N, nkv, d, generator=g), torch.randn(N, nkv, d, generator=g)
    q = torch.randn(1, nq, d, generator=g) * 30.0  # raw scores of hundreds: uncapped, one key would take everything
    k, v, q = (t.to(dtype).float() for t in (k, v, q))
    got = _attend(q, k, v, [N - 1], page, nq, nkv, d, 1.0, 2.0, None, dtype)
    want = _plain_attend(q, k, v, [N - 1], nq, nkv, 1.0, 2.0, None)
    assert _rel(got, want) < TOL[dtype]
    hard = _plain_attend(q, k, v, [N - 1], nq, nkv, 1.0, 0.0, None)
    assert _rel(got, hard) > 0.2  # the cap is not a no-op here
    # per-head sinks: head 0's sink dwarfs every score, head 1's is negligible
    q1 = (torch.randn(1, nq, d, generator=g) * 0.3).to(dtype).float()
    sinks = torch.tensor([12.0, -20.0])
    got = _attend(q1, k, v, [N - 1], page, nq, nkv, d, 1.0, 0.0, sinks, dtype)
    free = _plain_attend(q1, k, v, [N - 1], nq, nkv, 1.0, 0.0, None)
    assert float(got[0, 0].abs().max()) < 1e-2 * float(free[0, 0].abs().max()) + 1e-3
    assert _rel(got[0, 1], free[0, 1]) < TOL[dtype]
    assert _rel(got, _plain_attend(q1, k, v, [N - 1], nq, nkv, 1.0, 0.0, sinks)) < TOL[dtype]


# ---------------------------------------------------------------------------
# rotation table, projections' aftermath, small kernels


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq, nkv, d, e, rot, unit, biased", [(4, 2, 24, 16, 8, True, True), (3, 1, 16, 20, 16, False, False), (2, 2, 64, 64, 32, True, False),
                                                           (1, 1, 10, 6, 0, True, True), (2, 1, 128, 128, 64, True, True)])
def test_bias_rotation_unit_norm_and_store(dtype, nq, nkv, d, e, rot, unit, biased):
    from tokensprint_b200 import ops
    from tokensprint_b200.parts.position import scaled_frequencies

    T, eps = 19, 1e-5
    g = torch.Generator().manual_seed(d + e)
    n = nq * d + nkv * d + nkv * e
    proj = torch.randn(T, n + 5, generator=g).to(dtype)
    positions = [0, 1, 2, 3, 40, 41, 999, 1000, 5000, 5001, 7, 8, 9, 10, 11, 12, 13, 14, 15]
    bias = [torch.randn(w, generator=g) if biased else None for w in (nq * d, nkv * d, nkv * e)]
    table, freq, mag = None, None, 1.0
    if rot:
        freq, mag = scaled_frequencies(rot, 10000.0, {"kind": "yarn", "factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0})
        table = ops.rope_table(_i32(positions), _dev(freq), mag, T)
        ang = torch.tensor(positions, dtype=torch.float64)[:, None] * freq[None]
        assert torch.allclose(table[..., 0].cpu().double(), mag * torch.cos(ang), atol=2e-7)
        assert torch.allclose(table[..., 1].cpu().double(), mag * torch.sin(ang), atol=2e-7)
    D = max(d, e) if dtype == torch.float32 else -(-max(d, e) // 16) * 16
    q_out = torch.empty((T, nq, D), device="cuda", dtype=dtype)
    k_dst = torch.full((T + 4, nkv, D), float("nan"), device="cuda", dtype=dtype)
    v_dst = torch.full((T + 4, nkv, D), float("nan"), device="cuda", dtype=dtype)
    slots = [(3 * t + 1) % (T + 4) if t != 5 else -1 for t in range(T)]
    ops.qkv_prepare(_dev(proj), 0, nq * d, nq * d + nkv * d, *[None if b is None else _dev(b) for b in bias], table, unit, eps, q_out, k_dst, v_dst,
                    _i32(slots), nq, nkv, d, e, D)
    p = proj.double()
    q = p[:, :nq * d] + (bias[0].double() if biased else 0)
    k = p[:, nq * d:nq * d + nkv * d] + (bias[1].double() if biased else 0)
    v = p[:, nq * d + nkv * d:n] + (bias[2].double() if biased else 0)
    q, k = q.reshape(T, nq, d), k.reshape(T, nkv, d)
    if rot:
        q, k = plain.rotate_halves(q, positions, freq, mag), plain.rotate_halves(k, positions, freq, mag)
    if unit:
        q, k = plain.unit_rms(q, eps), plain.unit_rms(k, eps)
    tol = 2e-6 if dtype == torch.float32 else 1e-2
    assert _rel(q_out[..., :d], q) < tol and float(q_out[..., d:].float().abs().sum()) == 0.0
    for t in range(T):
        if slots[t] >= 0:
            assert _rel(k_dst[slots[t], :, :d], k[t]) < tol and _rel(v_dst[slots[t], :, :e], v[t].reshape(nkv, e)) < tol
            assert float(k_dst[slots[t], :, d:].float().abs().sum()) == 0.0 and float(v_dst[slots[t], :, e:].float().abs().sum()) == 0.0
    untouched = [s for s in range(T + 4) if s not in slots]
    assert bool(torch.isnan(k_dst[untouched].float()).all())


def test_gate_rows_weighted_sum_scale_and_float32_rows():
    from tokensprint_b200 import ops

    g = torch.Generator().manual_seed(8)
    for dtype in DTYPES:
        a, gate = torch.randn(7, 3, 16, generator=g).to(dtype), torch.randn(7, 40, generator=g).to(dtype)
        out = torch.empty((7, 30), device="cuda", dtype=dtype)
        ops.gate_rows(_dev(a), _dev(gate)[:, 5:35], out, 3, 10, 16)
        want = (a[..., :10].double().reshape(7, 30) * torch.sigmoid(gate[:, 5:35].double()))
        assert _rel(out, want) < (1e-6 if dtype == torch.float32 else 1e-2)
        xs = [torch.randn(9, 33, generator=g).to(dtype) for _ in range(3)]
        out = torch.empty((9, 33), device="cuda", dtype=dtype)
        ops.weighted_sum([_dev(x) for x in xs], [0.7, -1.3, 2.0], out)
        assert _rel(out, 0.7 * xs[0].double() - 1.3 * xs[1].double() + 2.0 * xs[2].double()) < (1e-6 if dtype == torch.float32 else 1e-2)
        x, w, b = torch.randn(11, 70, generator=g).to(dtype), torch.randn(5, 70, generator=g), torch.randn(5, generator=g)
        out = torch.empty((11, 5), device="cuda", dtype=torch.float32)
        ops.rows_dot_f32(_dev(x), _dev(w), _dev(b), out)
        assert _rel(out, x.double() @ w.double().T + b.double()) < 2e-6
    x = torch.randn(13, 21, generator=g)
    y = _dev(x.clone())
    ops.scale_rows(y, 0.375)
    assert torch.equal(y.cpu(), x * 0.375)
