"""Vasosun through the engine against the plain model, under every way of cutting and batching:
each request whole; most of it in one step and its last tokens one by one; in portions down to
two tokens; mixed, with so few pages and slots that both are used again; long decoding with and
without graphs; greedy generation through the entry point and the scheduler; the trace runner as
a program.

The float32 runs use sharpened queries (the softmax picks few keys, so one wrong key, a window
that is one position off, a lost kept input or a state that was not carried moves the logits far
beyond the tolerance).  The bfloat16 runs use the plain ones, and give every routed feed-forward a
small share of the stream: a router is a step function of its input, and a run in bfloat16 now and
then chooses another expert than the float64 model (the routed layer itself is held to the plain
one on its own in tests/test_vasosun_parts_gpu.py, where both read the same rows)."""

import pytest
import torch

from tests.plain import vasosun_plain as plain
from tests.replay_helpers import first_bad, replay_in_process, trace_decode_tail, trace_mixed, trace_portions, trace_whole, worst_error
from tests.vasosun_configs import VAS, random_ids, vasosun_weights, write_vasosun_folder

pytestmark = pytest.mark.gpu

# Largest allowed |engine - plain| relative to the largest |logit| of the sequence.
TOLERANCE = {"float32": 1e-4, "bfloat16": 8e-2}
SHARP = {"float32": 3.0, "bfloat16": 1.0}
ROUTED_SHARE = {"float32": 1.0, "bfloat16": 0.02}
LENGTHS = {"a": [1, 5, 17, 64, 100, 131], "b": [2, 9, 33, 90, 150], "c": [3, 26, 70, 129, 190], "d": [1, 2, 31, 77, 140]}
SEEDS = {"a": 71, "b": 72, "c": 73, "d": 74}
CASES = [("a", 16), ("b", 16), ("c", 16), ("d", 16), ("a", 8), ("c", 32), ("b", 256), ("d", 64)]


class Oracle:
    def __init__(self, cfg, weights):
        self.cfg, self.weights, self._cache = cfg, weights, {}

    def logits(self, ids):
        key = tuple(ids)
        if key not in self._cache:
            self._cache[key] = plain.forward_logits(ids, self.weights, self.cfg)
        return self._cache[key]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for tag, cfg in VAS.items():
        requests = {f"r{i}": random_ids(cfg, n, 1000 * SEEDS[tag] + i) for i, n in enumerate(LENGTHS[tag])}
        for dtype, sharp in SHARP.items():
            weights = vasosun_weights(cfg, SEEDS[tag], sharp=sharp, routed_share=ROUTED_SHARE[dtype])
            folder = write_vasosun_folder(tmp_path_factory.mktemp(f"vas_{tag}_{dtype}"), cfg, weights)
            out[tag, dtype] = (folder, cfg, requests, Oracle(cfg, weights))
    return out


def _replayer(folder, dtype, max_tokens, page_size=16, max_live=4, **kw):
    from tokensprint_b200.engine.replay import TraceReplayer

    r = TraceReplayer.from_folder(folder, dtype, max_tokens, page_size=page_size, max_live=max_live, **kw)
    r.runner.poison_freed_pages = True
    return r


def _check(got, requests, oracle, dtype, what):
    tol = TOLERANCE[dtype]
    worst, where = worst_error(got, requests, oracle)
    bad = first_bad(got, requests, oracle, tol)
    assert bad is None, f"{what}: first wrong token at request {bad[0]} position {bad[1]} (error {bad[2]:.3g}); worst {worst:.3g} at {where}"
    assert len(got) == sum(len(v) for v in requests.values()), f"{what}: logits are missing"


def _same(first, second, dtype, what):
    over = [key for key, row in first.items() if float(abs(row - second[key]).max()) > TOLERANCE[dtype] * float(abs(row).max())]
    assert not over, f"{what} changes {over[:5]}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag, page", CASES)
def test_whole(models, tag, page, dtype):
    folder, cfg, requests, oracle = models[tag, dtype]
    _check(replay_in_process(_replayer(folder, dtype, 256, page), trace_whole(requests)), requests, oracle, dtype, "whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag, page", CASES)
def test_decode_tail(models, tag, page, dtype):
    """The last 40 tokens one by one (more than the shortest windows): prefill against token-by-token
    decoding through pages, kept inputs and states."""
    folder, cfg, requests, oracle = models[tag, dtype]
    _check(replay_in_process(_replayer(folder, dtype, 256, page), trace_decode_tail(requests, 40)), requests, oracle, dtype, "decode tail")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag, page", CASES)
def test_portions(models, tag, page, dtype):
    """Portions shorter than the convolutions' taps stand beside long ones: the kept inputs of both
    sublayers of every layer, the delta states and the token before a portion are carried over every cut."""
    folder, cfg, requests, oracle = models[tag, dtype]
    _check(replay_in_process(_replayer(folder, dtype, 256, page), trace_portions(requests)), requests, oracle, dtype, "portions")
    sizes = (2, 2, 3, 2, 31, 2, 16, 1, 2, 17, 2)
    _check(replay_in_process(_replayer(folder, dtype, 256, page), trace_portions(requests, sizes)), requests, oracle, dtype, "small portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag, page", CASES)
def test_mixed_with_pages_and_slots_used_again(models, tag, page, dtype):
    folder, cfg, requests, oracle = models[tag, dtype]
    many = dict(requests)
    many.update({k + "x": v for k, v in requests.items()})
    max_tokens = {"a": 320, "b": 384, "c": 456, "d": 384}[tag]
    steps = trace_mixed(many, max_tokens, seed=11, max_live=3)
    replayer = _replayer(folder, dtype, max_tokens, page, max_live=3)
    got = replay_in_process(replayer, steps)
    cm = replayer.runner.cache_manager
    for pool in cm.pools:
        assert pool.num_free == pool.num_pages, "pages were lost"
    if cm.pools and page < 256:
        assert sum(-(-len(v) // page) for v in many.values()) > cm.pools[0].num_pages, "pages were not used again"
    assert len(many) > replayer.runner.num_slots, "slots were not used again"
    _check(got, many, oracle, dtype, "mixed")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", sorted(VAS))
def test_batches_of_unequal_requests_against_each_alone(models, tag, dtype):
    """The same positions alone and in a batch of unequal requests: equal beyond rounding."""
    folder, cfg, requests, oracle = models[tag, dtype]
    alone = replay_in_process(_replayer(folder, dtype, 512), trace_whole(requests))
    together = replay_in_process(_replayer(folder, dtype, 640, max_live=8), [
        {"step": 0, "entries": [{"id": k, "tokens": v, "want": list(range(len(v)))} for k, v in requests.items()], "end": list(requests)}])
    _same(alone, together, dtype, "batching")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["a", "b"])
def test_long_decoding_with_graphs_and_without(models, tag, dtype):
    """One prompt token, then more than a hundred tokens one by one (the windows of 20, 7 and 33 positions
    pass over decoded tokens many times), beside a second request that decodes too."""
    folder, cfg, requests, oracle = models[tag, dtype]
    reqs = {"p": requests["r4"][:1] + requests["r3"] + requests["r2"], "q": requests["r4"]}
    first = min(90, len(reqs["q"]) - 1)
    steps = [{"step": 0, "entries": [{"id": "p", "tokens": reqs["p"][:1], "want": [0]}, {"id": "q", "tokens": reqs["q"][:first], "want": list(range(first))}], "end": []}]
    for t in range(1, len(reqs["p"])):
        entries = [{"id": "p", "tokens": [reqs["p"][t]], "want": [0]}]
        if first + t - 1 < len(reqs["q"]):
            entries.append({"id": "q", "tokens": [reqs["q"][first + t - 1]], "want": [0]})
        steps.append({"step": t, "entries": entries, "end": []})
    results = []
    for graphs in (False, True):
        replayer = _replayer(folder, dtype, 512, graphs=graphs, max_model_len=256)
        got = replay_in_process(replayer, steps)
        _check(got, reqs, oracle, dtype, f"long decoding (graphs {graphs})")
        if graphs and dtype == "bfloat16":
            assert replayer.runner._graphs, "decode steps did not go through a graph"
        results.append(got)
    _same(results[0], results[1], dtype, "replaying graphs")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_request_whole_decoded_and_in_portions(tmp_path, dtype):
    """1,200 tokens: positions far beyond the `original` length, a window of 200 positions that passes over
    prompt and decoded tokens, temperatures that step a dozen times, prompt attention over hundreds of keys,
    decoded tokens whose keys are split over several CTAs, the delta state through all of it, with graphs and without."""
    from tests.vasosun_configs import VAS_LONG as cfg

    ids = random_ids(cfg, 1200, 7)
    reqs = {"r": ids}
    weights = vasosun_weights(cfg, 77, sharp=SHARP[dtype], routed_share=ROUTED_SHARE[dtype])
    folder = write_vasosun_folder(tmp_path / "long", cfg, weights)
    oracle = Oracle(cfg, weights)
    runs = [("whole", trace_whole(reqs), False), ("decode tail", trace_decode_tail(reqs, 230), False),
            ("decode tail, graphs", trace_decode_tail(reqs, 80), True), ("portions", trace_portions(reqs, (300, 2, 520, 64, 3, 700, 17)), False)]
    for what, steps, graphs in runs:
        replayer = _replayer(folder, dtype, 2048, graphs=graphs, max_model_len=2048)
        _check(replay_in_process(replayer, steps), reqs, oracle, dtype, what)


def _plain_greedy(weights, cfg, prompt, steps):
    ids = list(prompt)
    for _ in range(steps):
        ids.append(int(torch.argmax(plain.forward_logits(ids, weights, cfg)[-1])))
    return ids[len(prompt):]


@pytest.mark.parametrize("overlap", [True, False])
@pytest.mark.parametrize("eager", [True, False])
@pytest.mark.parametrize("tag", ["a", "b", "d"])
def test_greedy_generation_through_the_entry_point(models, tag, eager, overlap):
    """The scheduler cuts prompts into chunks of 24 tokens, batches them with decoding requests and
    hands decoded tokens on without the host seeing them (overlap); pages, kept inputs, states and the
    token before follow all of that, and slots are used again (four prompts, three at a time)."""
    from tokensprint_b200.config.engine_config import Config, SamplingParams
    from tokensprint_b200.engine.llm_engine import LLMEngine
    from tokensprint_b200.models.api import load_model

    folder, cfg, requests, oracle = models[tag, "float32"]
    prompts = [requests[k][:n] for k, n in (("r1", 5), ("r2", 17), ("r3", 50), ("r4", 64))]
    want = [_plain_greedy(oracle.weights, cfg, p, 12) for p in prompts]
    model, _ = load_model(folder, device="cuda", dtype="float32")
    engine = LLMEngine(model, Config(model=str(folder), max_model_len=256, num_kvcache_blocks=48, max_num_batched_tokens=24, max_num_seqs=3,
                                     chunked_prefill=True, dtype="float32", enforce_eager=eager, overlap_steps=overlap))
    got = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True), use_tqdm=False)
    assert got == want
    cm = engine.model_runner.cache_manager
    cm.check_invariants()
    assert all(cm.pages_in_use(g) == 0 for g in range(len(cm.pools)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_trace_runner_as_a_program(models, tmp_path, dtype):
    """bin/trace_run over stdin and stdout with a Vasosun folder: two requests, a portion of one beside single
    tokens of the other, a step in which nothing is wanted, files in --out, `done <step>` after every step."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    import numpy as np

    folder, cfg, requests, oracle = models["a", dtype]
    p, q = requests["r4"], requests["r2"]
    steps = [
        {"step": 0, "entries": [{"id": "p", "tokens": p[:40], "want": [0, 39]}], "end": []},
        {"step": 1, "entries": [{"id": "q", "tokens": q[:15], "want": [14]}, {"id": "p", "tokens": p[40:41], "want": [0]}], "end": []},
        {"step": 2, "entries": [{"id": "p", "tokens": p[41:43], "want": []}], "end": []},
        {"step": 3, "entries": [{"id": "q", "tokens": q[15:], "want": [1]}, {"id": "p", "tokens": p[43:], "want": [len(p) - 44]}], "end": ["p", "q"]},
    ]
    root = Path(__file__).resolve().parents[1]
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out), "--max-tokens", "192"],
        input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
    assert sorted(f.name for f in out.iterdir()) == ["0.f32", "1.f32", "3.f32"]
    want_p, want_q = oracle.logits(p).numpy(), oracle.logits(q).numpy()
    got = {n: np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, cfg["vocab"]) for n in (0, 1, 3)}
    pairs = [(got[0][0], want_p[0]), (got[0][1], want_p[39]), (got[1][0], want_q[14]), (got[1][1], want_p[40]),
             (got[3][0], want_q[16]), (got[3][1], want_p[-1])]
    for g, w in pairs:
        assert np.abs(g - w).max() < TOLERANCE[dtype] * max(np.abs(want_p).max(), np.abs(want_q).max())
