"""Vasosun models of random shapes through the engine: widths, head counts, key and value widths,
latents and rotated parts that are multiples of nothing in particular, any order of the three
mixers (a reader of cached rows wherever an earlier layer caches some of its shape), windows from a
few positions to none, one to five taps, delta layers with one tap, experts of which all are chosen,
no identity experts or several, layers without a feed-forward.  Each model runs whole, in portions,
with a decoded tail and mixed with pages and slots used again, in float32 against the float64 plain
model (sharpened queries), and in bfloat16 for finite logits that agree between the cuttings (the
routed layers get a small share of the stream there: a router is a step function of its input)."""

import random

import numpy as np
import pytest

from tests.plain import vasosun_plain as plain
from tests.replay_helpers import replay_in_process, trace_decode_tail, trace_mixed, trace_portions, trace_whole
from tests.vasosun_configs import random_ids, vasosun_weights, write_vasosun_folder

pytestmark = pytest.mark.gpu


def random_config(rng: random.Random) -> dict:
    width = rng.choice([40, 56, 64, 100, 128, 136, 200, 256])
    layers, latents = [], []  # latents: (layer, mixer) of the layers that cache rows of their own

    def attention():
        kv = rng.choice([1, 2, 3, 4])
        m = {"heads": kv * rng.choice([1, 2, 4]), "kv_heads": kv, "dim": rng.choice([6, 8, 16, 24, 32, 48, 64, 80, 128]),
             "vdim": rng.choice([4, 8, 16, 20, 32, 64, 128]), "scale": rng.choice([0.05, 0.1, 0.2])}
        if rng.random() < 0.85:
            m["mask"] = {"size": rng.choice([1, 2, 5, 16, 17, 33, 64, 100, 500])}
        if rng.random() < 0.85:
            m["q_temp"] = {"coef": rng.choice([0.1, 0.5, 2.0]), "every": rng.choice([1, 2, 7, 16, 64, 1000])}
        return {"type": "attention", "mixer": m}

    def latent():
        if latents and rng.random() < 0.5:  # a reader: the source's latent width, rotated part and rotation; the rest its own
            j, src = rng.choice(latents)
            m = dict(src, heads=rng.choice([1, 2, 3, 4, 8]), dim=rng.choice([2, 8, 16, 24, 32]), vdim=rng.choice([4, 8, 12, 32, 64]),
                     q_rank=rng.choice([6, 16, 24, 48]), scale=rng.choice([0.05, 0.1, 0.2]), kv_from=j)
            return {"type": "latent_attention", "mixer": m}
        rot_dim = rng.choice([2, 4, 8, 16, 32, 48])
        dims = rng.choice(range(2, rot_dim + 1, 2)) if rng.random() < 0.3 else rot_dim
        rot = {"base": rng.choice([100.0, 10000.0, 1e6]), "dims": dims}
        if rng.random() < 0.6:
            rot["scaling"] = {"factor": rng.choice([2.0, 4.0, 8.0]), "original": rng.choice([16, 32, 64, 4096]),
                              "fast": rng.choice([4.0, 8.0, 32.0]), "slow": rng.choice([0.5, 1.0, 2.0])}
        m = {"heads": rng.choice([1, 2, 3, 4, 6, 8]), "dim": rng.choice([2, 8, 16, 24, 32, 40, 64]), "rot_dim": rot_dim,
             "vdim": rng.choice([8, 12, 16, 32, 64]), "kv_rank": rng.choice([8, 16, 20, 32, 48, 64, 96, 128]),
             "q_rank": rng.choice([6, 16, 24, 48, 96]), "scale": rng.choice([0.05, 0.1, 0.2]), "rot": rot}
        latents.append((len(layers), m))
        return {"type": "latent_attention", "mixer": m}

    def delta():
        kv = rng.choice([1, 2, 3])
        return {"type": "delta", "mixer": {"heads": kv * rng.choice([1, 2, 4]), "kv_heads": kv, "dim": rng.choice([3, 8, 12, 16, 32, 40, 64, 96, 128]),
                                           "vdim": rng.choice([4, 8, 10, 16, 32, 64]), "conv": rng.choice([1, 2, 3, 4, 5])}}

    for _ in range(rng.randint(1, 6)):
        k = rng.random()
        if k < 0.2:
            mlp = None
        elif k < 0.5:
            mlp = {"kind": "dense", "ff": rng.choice([24, 64, 100, 256])}
        else:
            experts, identity = rng.choice([1, 2, 4, 6, 12, 33]), rng.choice([0, 0, 1, 2, 5])
            mlp = {"kind": "moe", "expert": {"ff": rng.choice([8, 24, 36, 64])},
                   "router": {"experts": experts, "identity": identity, "top": rng.randint(1, min(experts + identity, 4))}}
        layers.append(dict(rng.choice([attention, latent, delta])(), mlp=mlp))
    return {"architecture": "Vasosun", "vocab": rng.choice([50, 211, 333, 1000]), "width": width, "norm": {"eps": rng.choice([1e-5, 1e-6])},
            "canon": {"taps": rng.choice([1, 2, 3, 4, 5])}, "logit_softcap": rng.choice([5.0, 30.0, 100.0]),
            "embedding": {"bigram": {"buckets": rng.choice([7, 97, 601, 4099]), "mul_prev": rng.choice([1, 31, 113, 1000003]), "mul_cur": rng.choice([1, 5, 13])}},
            "layers": layers}


@pytest.mark.parametrize("seed", range(10))
def test_random_model_in_every_cutting(tmp_path, seed):
    from tokensprint_b200.engine.replay import TraceReplayer

    cfg = random_config(random.Random(2000 + seed))
    requests = {f"r{i}": random_ids(cfg, n, seed * 100 + i) for i, n in enumerate([1, 7, 40, 90, 131])}
    for dtype, sharp in (("float32", 2.0), ("bfloat16", 1.0)):
        weights = vasosun_weights(cfg, seed, sharp=sharp, routed_share=1.0 if dtype == "float32" else 0.01)
        folder = write_vasosun_folder(tmp_path / dtype, cfg, weights)
        want = {k: plain.forward_logits(v, weights, cfg).numpy() for k, v in requests.items()}
        runs = {}
        for name, steps, max_tokens in (("whole", trace_whole(requests), 512), ("portions", trace_portions(requests), 512),
                                        ("tail", trace_decode_tail(requests, 8), 512), ("mixed", trace_mixed(requests, 320, seed=seed, max_live=3), 320)):
            replayer = TraceReplayer.from_folder(folder, dtype, max_tokens, page_size=16, max_live=3)
            replayer.runner.poison_freed_pages = True
            runs[name] = got = replay_in_process(replayer, steps)
            assert len(got) == sum(len(v) for v in requests.values())
            for (rid, pos), row in got.items():
                assert np.isfinite(row).all(), f"{dtype} {name}: request {rid} position {pos} is not finite\n{cfg}"
                if dtype == "float32":
                    err = float(np.abs(row - want[rid][pos]).max() / np.abs(want[rid]).max())
                    assert err < 3e-4, f"float32 {name}: request {rid} position {pos}: error {err:.3g}\n{cfg}"
        tol = 1e-4 if dtype == "float32" else 5e-2
        for name in ("portions", "tail", "mixed"):
            for key, row in runs["whole"].items():
                scale = float(np.abs(want[key[0]]).max())
                assert float(np.abs(row - runs[name][key]).max()) <= tol * scale, f"{dtype}: whole and {name} differ at {key}\n{cfg}"
