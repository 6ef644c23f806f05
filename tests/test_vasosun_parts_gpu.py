"""The mechanisms of Vasosun one at a time: each kernel and each mixer part against the plain
function of the same mechanism, whole prompts, portions down to one token, batches of unequal
sequences with slots and pages in any order and used again; inputs made so that a key just inside
or just outside a window, a far key, a lost kept input or a state that was not carried shows far
beyond rounding."""

import pytest
import torch

from tests.plain import vasosun_plain as plain
from tests.vasosun_configs import VAS, VAS_LONG, vasosun_weights

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


def _rand(shape, seed):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed))


# ---------------------------------------------------------------------------
# kernels alone


def _batch(lengths):
    cu = [0]
    for n in lengths:
        cu.append(cu[-1] + n)
    seq = [b for b, n in enumerate(lengths) for _ in range(n)]
    return _i32(cu), _i32(seq)


@pytest.mark.parametrize("taps", [1, 2, 3, 5])
@pytest.mark.parametrize("mode", ["add_input", "silu"])
@pytest.mark.parametrize("in_dtype, out_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.float32), (torch.bfloat16, torch.bfloat16)])
def test_causal_conv_in_portions_and_batches(taps, mode, in_dtype, out_dtype):
    """Three sequences of unequal length go through in portions of 1, 2 and more tokens, side by side in
    one launch, in slots given in any order; a fourth takes over a slot that was used before."""
    from tokensprint_b200 import ops

    C = 37
    w = _rand((C, taps), 1) * 0.7
    seqs = {"a": _rand((23, C), 2), "b": _rand((9, C), 3), "c": _rand((40, C), 4), "d": _rand((6, C), 5)}
    seqs = {k: v.to(in_dtype).float() for k, v in seqs.items()}

    def want(x):
        c = plain.causal_conv(x.double(), w.double())
        return x.double() + c if mode == "add_input" else plain.silu(c)

    state = torch.full((3, 5 + max(taps - 1, 0) * C), float("nan"), device="cuda")  # a view with a row stride, as a mixer's slot gives it
    view = state[:, 5:] if taps > 1 else None
    slot_of, done, got = {"a": 2, "b": 0, "c": 1}, {k: 0 for k in seqs}, {k: [] for k in seqs}
    for k in slot_of:
        state[slot_of[k]].zero_()
    plan = [{"a": 1, "b": 2, "c": 7}, {"a": 2, "c": 1}, {"b": 7, "a": 20, "c": 32}, {"d": 1}, {"d": 2}, {"d": 3}]
    for step in plan:
        if "d" in step and "d" not in slot_of:  # the request in slot 0 has ended: its slot is zeroed and used again
            slot_of["d"] = slot_of.pop("b")
            state[slot_of["d"]].zero_()
        names = sorted(step)
        rows = torch.cat([seqs[k][done[k]:done[k] + step[k]] for k in names])
        cu, seq = _batch([step[k] for k in names])
        out = torch.empty(rows.shape, device="cuda", dtype=out_dtype)
        ops.causal_conv(_dev(rows, in_dtype), _dev(w.t().contiguous()), None, view, _i32([slot_of[k] for k in names]), cu, seq, len(names), out,
                        activation="silu" if mode == "silu" else None, add_input=mode == "add_input")
        at = 0
        for k in names:
            got[k].append(out[at:at + step[k]].float().cpu())
            at += step[k]
            done[k] += step[k]
    for k, x in seqs.items():
        assert done[k] == x.shape[0]
        assert _rel(torch.cat(got[k]), want(x)) < (1e-5 if out_dtype == torch.float32 else 1e-2), (k, taps, mode)


DELTA_SHAPES = [(1, 1, 7, 5), (6, 3, 20, 10), (2, 2, 64, 64), (4, 2, 128, 32), (3, 3, 9, 14), (2, 1, 256, 20)]


def _delta_inputs(H, G, d, e, T, seed):
    x = _rand((T, 2 * G * d + H * e), seed)
    gates = torch.cat([_rand((T, H), seed + 1), _rand((T, H), seed + 2) - 2.0], dim=1)
    a_log, dt_bias = 0.3 + 0.3 * _rand((H,), seed + 3), -1.0 + 0.5 * _rand((H,), seed + 4)
    return x, gates, a_log, dt_bias


def _delta_plain(x, gates, a_log, dt_bias, H, G, d, e):
    T = x.shape[0]
    x, gates = x.double(), gates.double()
    q = plain.unit_length(x[:, :G * d].view(T, G, d)) * d ** -0.5
    k = plain.unit_length(x[:, G * d:2 * G * d].view(T, G, d))
    v = x[:, 2 * G * d:].view(T, H, e)
    beta = torch.sigmoid(gates[:, :H])
    decay = torch.exp(-torch.exp(a_log.double()) * plain.softplus(gates[:, H:] + dt_bias.double()))
    return torch.cat([plain.delta_recurrence(q[:, a // (H // G)], k[:, a // (H // G)], v[:, a], decay[:, a], beta[:, a]) for a in range(H)], -1)


def _delta_run(x, gates, a_log, dt_bias, state, slots, lengths, H, G, d, e):
    from tokensprint_b200 import ops

    cu, _ = _batch(lengths)
    out = torch.empty((x.shape[0], H * e), device="cuda")
    ops.delta_scan(_dev(x), 0, G * d, 2 * G * d, _dev(gates), _dev(a_log), _dev(dt_bias), state, _i32(slots), cu, out, len(lengths), H, G, d, e,
                   d ** -0.5, 1e-6)
    return out.cpu()


@pytest.mark.parametrize("H, G, d, e", DELTA_SHAPES)
def test_delta_scan_whole_in_portions_and_token_by_token(H, G, d, e):
    T = 150
    x, gates, a_log, dt_bias = _delta_inputs(H, G, d, e, T, 10 * d + e)
    want = _delta_plain(x, gates, a_log, dt_bias, H, G, d, e)
    floats = H * d * e
    for sizes in ([T], [1, 2, 7, 1, 33, 2, 64, 3, 37], [1] * 40 + [110]):
        state = torch.zeros((4, floats + 3), device="cuda")  # a row stride that is no multiple of four
        got, at = [], 0
        for n in sizes:
            got.append(_delta_run(x[at:at + n], gates[at:at + n], a_log, dt_bias, state, [2], [n], H, G, d, e))
            at += n
        assert _rel(torch.cat(got), want) < 3e-5, (sizes[:3], H, G, d, e)
        assert float(state[[0, 1, 3]].abs().max()) == 0.0 and float(state[2, floats:].abs().max()) == 0.0  # nobody else's slot, nothing behind the state


@pytest.mark.parametrize("H, G, d, e", [(6, 3, 20, 10), (2, 2, 64, 64)])
def test_delta_scan_many_sequences_side_by_side_against_each_alone(H, G, d, e):
    """Forty sequences of unequal length (one of them empty: a padded lane) in one launch, their slots in
    any order: each as it is alone."""
    lengths = [(7 * i) % 23 + (0 if i == 5 else 1) for i in range(40)]
    lengths[5] = 0
    data = [_delta_inputs(H, G, d, e, max(n, 1), 100 + i) for i, n in enumerate(lengths)]
    a_log, dt_bias = data[0][2], data[0][3]
    state = torch.zeros((40, H * d * e), device="cuda")
    slots = [(3 * i) % 40 for i in range(40)]  # 3 and 40 have no common factor: every slot once
    state[slots[5]] = 7.0  # the empty lane's slot must stay as it is
    x = torch.cat([data[i][0][:n] for i, n in enumerate(lengths)])
    gates = torch.cat([data[i][1][:n] for i, n in enumerate(lengths)])
    got = _delta_run(x, gates, a_log, dt_bias, state, slots, lengths, H, G, d, e)
    at = 0
    for i, n in enumerate(lengths):
        if n:
            want = _delta_plain(data[i][0][:n], data[i][1][:n], a_log, dt_bias, H, G, d, e)
            assert _rel(got[at:at + n], want) < 3e-5, i
        at += n
    assert float((state[slots[5]] - 7.0).abs().max()) == 0.0


def test_router_scores_correction_and_identity_combine():
    from tokensprint_b200 import ops

    T, W, E, ident, top = 50, 40, 6, 2, 3
    rows, router, corr = _rand((T, W), 1), _rand((E + ident, W), 2) * 0.4, _rand((E + ident,), 3) * 0.2
    s = torch.softmax(rows.double() @ router.double().T, -1)
    key = s + corr.double()
    want_ids = torch.topk(key, top, -1).indices
    ids = torch.empty((T, top), device="cuda", dtype=torch.int32)
    wts = torch.empty((T, top), device="cuda")
    ops.router(_dev(rows), _dev(router), top, False, ids, wts, score="softmax_all", correction=_dev(corr))
    margin = torch.topk(key, top + 1, -1).values
    clear = (margin[:, top - 1] - margin[:, top]) > 1e-5
    assert bool(clear.sum() > 40)
    assert torch.equal(ids.cpu().long()[clear].sort(-1).values, want_ids[clear].sort(-1).values)
    assert _rel(wts.cpu()[clear], torch.gather(s, 1, ids.cpu().long())[clear]) < 1e-5
    # the combine: pairs of identity experts read the input row, the others their expert's row; rows of pairs
    # without an expert hold whatever memory held (NaN here) and must not be read
    x, pair_out = _rand((T, W), 4), _rand((T * top, W), 5)
    identity = (ids.cpu() >= E).view(-1)
    poisoned = pair_out.clone()
    poisoned[identity] = float("nan")
    out = torch.empty((T, W), device="cuda")
    ops.moe_combine(_dev(poisoned), None, out, top, wts.view(-1), ids=ids, num_experts=E, x=_dev(x))
    rows_used = torch.where(identity[:, None], x.repeat_interleave(top, 0), pair_out)
    want = (rows_used.double() * wts.cpu().double().view(-1, 1)).view(T, top, W).sum(1)
    assert _rel(out.cpu(), want) < 1e-5


def test_softcap_rows():
    from tokensprint_b200 import ops

    x = _rand((7, 33), 1) * 40
    y = _dev(x.clone())
    ops.softcap_rows(y, 12.5)
    assert _rel(y.cpu(), 12.5 * torch.tanh(x.double() / 12.5)) < 1e-6


# ---------------------------------------------------------------------------
# parts


def _layer_parts(cfg, layer, dtype, seed, sharp):
    """Mixer and feed-forward of one layer, built from the engine's own specification, with the tests' weights."""
    from tokensprint_b200.models.vasosun import VasosunConfig, build_vasosun_spec
    from tokensprint_b200.parts.base import BuildContext, build_part

    W = vasosun_weights(cfg, seed, sharp=sharp)
    params = build_vasosun_spec(VasosunConfig.from_dict(cfg)).layers[layer].params
    ctx = BuildContext(torch.device("cuda"), dtype)
    parts = {}
    for kind, key in (("mixer", "mixer"), ("feed_forward", "feed_forward")):
        if params.get(key) is not None:
            part = build_part(kind, params[key], ctx)
            part.load({s.name: _dev(W[s.name], torch.float32 if s.role == "vector" else dtype) for s in part.tensor_specs()})
            parts[key] = part
    return parts, {k: v.double() for k, v in W.items()}


class Harness:
    """Pages and state slots for one mixer (and for mixers that read its pages), and steps of
    (sequence, its next n tokens) in any batch; pages come in a shuffled order and freed ones are used again first."""

    def __init__(self, mixer, dtype, page=16, num_pages=96, slots=5, seed=0, readers=()):
        self.mixers, self.dtype, self.page = [mixer, *readers], dtype, page
        need = mixer.cache_need()
        self.k = self.v = None
        if need.kind != "none":
            self.k = torch.full((num_pages, page, *need.k_row), float("nan"), device="cuda", dtype=dtype)
            self.v = None if need.v_row is None else torch.full((num_pages, page, *need.v_row), float("nan"), device="cuda", dtype=dtype)
        self.states = [None if m.cache_need().state_shape is None else torch.zeros((slots, *m.cache_need().state_shape), device="cuda")
                       for m in self.mixers]
        self.free_pages = torch.randperm(num_pages, generator=torch.Generator().manual_seed(seed)).tolist()
        self.pages, self.done, self.slot = {}, {}, {}
        self.free_slots = list(range(slots))[::-1]

    def end(self, name):
        self.free_pages = self.pages.pop(name, []) + self.free_pages
        self.free_slots.append(self.slot.pop(name))
        del self.done[name]

    def step(self, x_by_seq, which=0):
        """Runs mixer `which` (0: the one that fills the pages) on the given rows; a reader runs on positions that
        the writer has stored already (`advance` False then)."""
        from tokensprint_b200 import ops
        from tokensprint_b200.parts.base import GroupTables, LayerCache, StepContext

        names = sorted(x_by_seq, key=lambda n: (x_by_seq[n].shape[0] != 1, n))  # single tokens first, as the runner orders them
        pos, seq, cu, ctx, slots, slot_map, rows = [], [], [0], [], [], [], []
        for b, name in enumerate(names):
            n = x_by_seq[name].shape[0]
            if name not in self.done:
                self.done[name], self.pages[name] = [0] * len(self.mixers), []
                self.slot[name] = self.free_slots.pop()
                for st in self.states:
                    if st is not None:
                        st[self.slot[name]].zero_()
            start = self.done[name][which]
            while len(self.pages[name]) * self.page < start + n:
                self.pages[name].append(self.free_pages.pop(0))
            pos += range(start, start + n)
            seq += [b] * n
            cu.append(cu[-1] + n)
            ctx.append(start + n)
            slots.append(self.slot[name])
            slot_map += [self.pages[name][p // self.page] * self.page + p % self.page for p in range(start, start + n)]
            rows.append(x_by_seq[name])
            self.done[name][which] = start + n
        width = max(len(self.pages[n]) for n in names)
        table = [self.pages[n] + [-1] * (width - len(self.pages[n])) for n in names]
        T = cu[-1]
        lens = [x_by_seq[n].shape[0] for n in names]
        step = StepContext(num_tokens=T, num_seqs=len(names), token_ids=_i32([0] * T), positions=_i32(pos), seq_index=_i32(seq),
                           cu_seqlens_q=_i32(cu), context_lens=_i32(ctx), state_slots=_i32(slots),
                           groups=[GroupTables(_i32(sum(table, [])).view(len(names), width), _i32(slot_map))], page_size=self.page,
                           max_seqlen_q=max(lens), max_context_len=max(ctx), decode_only=all(n == 1 for n in lens),
                           decode_seqs=sum(1 for n in lens if n == 1))
        cache = LayerCache(group=0 if self.k is not None else -1, k_pages=self.k, v_pages=self.v, state=self.states[which], writes=which == 0)
        out = self.mixers[which].forward(_dev(torch.cat(rows).to(self.dtype)), step, cache)
        ops.flush_gemm_chain()
        return {name: out[cu[b]:cu[b + 1]].float().cpu() for b, name in enumerate(names)}


def _inputs(T, width, seed, dtype):
    return _rand((T, width), seed).to(dtype).float()  # what both sides read


def _in_portions(h, name, x, sizes, which=0):
    out, pos, i = [], 0, 0
    while pos < x.shape[0]:
        n = min(sizes[i % len(sizes)], x.shape[0] - pos)
        out.append(h.step({name: x[pos:pos + n]}, which)[name])
        pos, i = pos + n, i + 1
    return torch.cat(out)


def _plain_mixer(cfg, layer, W):
    entry, eps, p = cfg["layers"][layer], cfg["norm"]["eps"], f"l{layer}.mix."
    m = entry["mixer"]
    if entry["type"] == "attention":
        return lambda x: plain.window_attention(x, list(range(x.shape[0])), m, W, p)
    if entry["type"] == "delta":
        return lambda x: plain.delta_mixer(x, m, W, p, eps)
    raise ValueError(entry["type"])


OWN_CACHE = [(tag, i) for tag, cfg in sorted(VAS.items()) for i, l in enumerate(cfg["layers"]) if l["type"] != "latent_attention"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tag, layer", OWN_CACHE)
def test_attention_and_delta_mixers_in_every_cutting(tag, layer, dtype):
    """Whole, in portions down to one token, token by token over more positions than the window, and in a batch of
    unequal sequences whose pages and slots were used before, against the plain mechanism."""
    cfg = VAS[tag]
    parts, W = _layer_parts(cfg, layer, dtype, 21, 2.0)
    mixer, f = parts["mixer"], _plain_mixer(cfg, layer, W)
    xs = {name: _inputs(n, cfg["width"], 30 + i, dtype) for i, (name, n) in enumerate((("a", 75), ("b", 9), ("c", 41)))}
    want = {name: f(x.double()) for name, x in xs.items()}
    for page in (16, 8):
        h = Harness(mixer, dtype, page=page)
        assert _rel(h.step({"a": xs["a"]})["a"], want["a"]) < TOL[dtype], "whole"
        h.end("a")
        assert _rel(_in_portions(h, "a", xs["a"], (1, 2, 5, 1, 16, 2, 3)), want["a"]) < TOL[dtype], "portions"
        h.end("a")
        assert _rel(_in_portions(h, "a", xs["a"], (1,)), want["a"]) < TOL[dtype], "token by token"
        h.end("a")
        got = {name: [] for name in xs}
        for step in ({"a": 30, "b": 1, "c": 2}, {"a": 1, "b": 1}, {"a": 44, "b": 7, "c": 39}):
            at = {name: sum(t.shape[0] for t in got[name]) for name in step}
            for name, rows in h.step({name: xs[name][at[name]:at[name] + n] for name, n in step.items()}).items():
                got[name].append(rows)
        for name in xs:
            assert _rel(torch.cat(got[name]), want[name]) < TOL[dtype], f"batch, {name}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tag", ["a", "c"])
def test_a_key_at_the_windows_edge_and_a_far_key(tag, dtype):
    """One token's input is made ten times as large (its key and value then dominate wherever they are seen): the
    queries that have it just inside their window, just outside it, and far behind agree with the plain mechanism,
    in a prompt and token by token."""
    cfg = VAS[tag]
    layer = next(i for i, l in enumerate(cfg["layers"]) if l["type"] == "attention" and l["mixer"].get("mask"))
    size = cfg["layers"][layer]["mixer"]["mask"]["size"]
    parts, W = _layer_parts(cfg, layer, dtype, 22, 3.0)
    x = _inputs(3 * size + 5, cfg["width"], 40, dtype)
    loud = size // 2 + 3
    x[loud] *= 10.0
    want = plain.window_attention(x.double(), list(range(x.shape[0])), cfg["layers"][layer]["mixer"], W, f"l{layer}.mix.")
    quiet = x.clone()
    quiet[loud] /= 10.0
    base = plain.window_attention(quiet.double(), list(range(x.shape[0])), cfg["layers"][layer]["mixer"], W, f"l{layer}.mix.")
    moved = (want - base).abs().amax(-1)
    assert float(moved[loud + size - 1]) > 1e-3 and float(moved[loud + size]) == 0.0  # the last query that sees it, the first that does not
    for sizes in ((x.shape[0],), (loud + size - 2, 1, 1, 1, 1), (1,)):
        h = Harness(parts["mixer"], dtype, page=8)
        got = _in_portions(h, "s", x, sizes)
        assert _rel(got, want) < TOL[dtype], sizes
        assert _rel(got[loud + size - 2:loud + size + 2], want[loud + size - 2:loud + size + 2]) < TOL[dtype], "at the edge"


LATENT = [(tag, i) for tag, cfg in sorted(VAS.items()) for i, l in enumerate(cfg["layers"])
          if l["type"] == "latent_attention" and l["mixer"].get("kv_from") is None] + [("long", 1)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tag, layer", LATENT)
def test_latent_attention_and_the_layers_that_read_its_rows(tag, layer, dtype):
    """The layer that caches [latent ; rotated key part] and every layer that reads those rows with matrices of its
    own: whole, in portions, token by token; the readers run behind the writer on the same pages."""
    cfg = VAS_LONG if tag == "long" else VAS[tag]
    eps = cfg["norm"]["eps"]
    readers = [i for i, l in enumerate(cfg["layers"]) if l["type"] == "latent_attention" and l["mixer"].get("kv_from") == layer]
    built = {i: _layer_parts(cfg, i, dtype, 23, 2.0) for i in [layer] + readers}
    W = built[layer][1]
    T = 300 if tag == "long" else 70
    xs = {i: _inputs(T, cfg["width"], 50 + i, dtype) for i in [layer] + readers}
    pos = list(range(T))
    m = cfg["layers"][layer]["mixer"]
    c, kr = plain.latent_rows(xs[layer].double(), pos, m, W, f"l{layer}.mix.", eps)
    want = {i: plain.latent_attention(xs[i].double(), pos, cfg["layers"][i]["mixer"], W, f"l{i}.mix.", eps, c, kr) for i in xs}
    for sizes in ((T,), (1, 2, 7, 1, 33, 2), (1,)):
        h = Harness(built[layer][0]["mixer"], dtype, page=16, readers=[built[i][0]["mixer"] for i in readers])
        at, k, got = 0, 0, {i: [] for i in xs}
        while at < T:
            n = min(sizes[k % len(sizes)], T - at)
            for which, i in enumerate([layer] + readers):  # the writer first, as in the model's run order
                got[i].append(h.step({"s": xs[i][at:at + n]}, which)["s"])
            at, k = at + n, k + 1
            if sizes == (1,) and at >= 40:
                break
        for i in xs:
            rows = torch.cat(got[i])
            assert _rel(rows, want[i][:rows.shape[0]]) < TOL[dtype], (sizes, i)


ROUTED = [(tag, i) for tag, cfg in sorted(VAS.items()) for i, l in enumerate(cfg["layers"]) if l["mlp"] is not None and l["mlp"]["kind"] == "moe"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tag, layer", ROUTED)
def test_routed_experts_on_the_same_rows(tag, layer, dtype):
    """Engine and plain model read the same rows; tokens whose choice hangs on less than 1e-4 of a score are left out."""
    cfg = VAS[tag]
    parts, W = _layer_parts(cfg, layer, dtype, 24, 1.0)
    mlp, p = cfg["layers"][layer]["mlp"], f"l{layer}.mlp."
    for T in (1, 3, 70):
        x = _inputs(T, cfg["width"], 60 + T, dtype)
        got = parts["feed_forward"].forward(_dev(x.to(dtype)), None).float().cpu()
        want = plain.routed_ff(x.double(), mlp, W, p)
        s = torch.softmax(x.double() @ W[p + "router"].T, -1) + W[p + "correction"]
        top = mlp["router"]["top"]
        clear = torch.ones(T, dtype=torch.bool)
        if top < s.shape[1]:
            best = torch.topk(s, top + 1, -1).values
            clear = (best[:, top - 1] - best[:, top]) > 1e-4
        assert _rel(got[clear], want[clear]) < TOL[dtype], T
