"""The tests' own small Vasosun configurations and weights (no product code here).

The configurations differ from one another in every size and option: head counts and grouping
(every query head with its own keys, all with one), key widths against value widths, windows from
seven positions to none, query temperatures that step every few positions, latents of 20 to 64
entries with rotated parts that turn in full or in part, with stretched frequencies or plain ones,
layers that read the rows an earlier layer cached (one reader, two readers, not the neighbour),
delta layers with one head and with six, two to five taps, input convolutions of one tap (no kept
inputs) to five, layers without a feed-forward, dense ones, and routed experts with none, one or as
many identity experts as real ones, one to three choices per token.  Weights come from the tests'
integer-hash generator under the checkpoint's tensor names.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Optional

import torch

from tests.tiny_configs import seeded_normal


def _yarn(factor, original, fast, slow):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


def _att(heads, kv_heads, dim, vdim, scale, window, coef, every):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "q_temp": {"coef": coef, "every": every}}
    if window:
        m["mask"] = {"size": window}
    return {"type": "attention", "mixer": m}


def _lat(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, dims, scaling=None, kv_from=None):
    rot = {"base": base, "dims": dims}
    if scaling is not None:
        rot["scaling"] = scaling
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale, "rot": rot}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def _delta(heads, kv_heads, dim, vdim, conv):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, experts, identity, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}


def _layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


def _model(vocab, width, eps, taps, buckets, mul_prev, mul_cur, cap, layers):
    return {"architecture": "Vasosun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "canon": {"taps": taps},
            "embedding": {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}, "logit_softcap": cap, "layers": layers}


# all three mixers; a reader of cached rows that is not its source's neighbour; part of the rotated part turns; a layer
# without a feed-forward; routed experts with two, none and one identity expert
_A_ROT = (1000.0, 6, _yarn(4.0, 32, 8.0, 1.0))
VAS_A = _model(211, 96, 1e-5, 4, 97, 7, 13, 12.0, [
    _layer(_att(4, 2, 24, 16, 0.3, 20, 0.7, 8), _dense(40)),
    _layer(_lat(3, 10, 8, 12, 20, 14, 0.25, *_A_ROT), _moe(24, 5, 2, 3)),
    _layer(_delta(4, 2, 12, 10, 3), None),
    _layer(_lat(2, 6, 8, 9, 20, 10, 0.4, *_A_ROT, kv_from=1), _moe(16, 4, 0, 2)),
    _layer(_att(2, 2, 16, 32, 0.25, 7, 0.3, 3), _moe(8, 3, 1, 1)),
])

# input convolutions of one tap (nothing kept); the layers begin with a delta layer of one head with odd widths; one
# key/value head for five query heads; as many identity experts as real ones
VAS_B = _model(130, 72, 3e-6, 1, 61, 31, 1, 50.0, [
    _layer(_delta(1, 1, 7, 5, 2), _dense(20)),
    _layer(_att(5, 1, 12, 28, 0.2, 33, 1.0, 16), None),
    _layer(_delta(6, 3, 20, 10, 5), _moe(10, 3, 3, 2)),
])

# widths the tensor-core kernels take (heads of 64 and 128, latent 64 + 16, expert widths that are multiples of 8);
# two readers of the first layer's rows; whole rotated parts turn with plain frequencies; a layer that sees every earlier key
_C_ROT = (50000.0, 16, None)
VAS_C = _model(300, 128, 1e-6, 2, 509, 3, 5, 30.0, [
    _layer(_lat(4, 32, 16, 32, 64, 48, 0.15, *_C_ROT), _dense(64)),
    _layer(_att(4, 2, 64, 64, 0.125, 48, 0.5, 32), _moe(32, 8, 1, 2)),
    _layer(_lat(2, 16, 16, 64, 64, 32, 0.2, *_C_ROT, kv_from=0), _moe(64, 4, 2, 3)),
    _layer(_lat(4, 48, 16, 16, 64, 64, 0.12, *_C_ROT, kv_from=0), None),
    _layer(_delta(2, 2, 64, 64, 4), _dense(96)),
    _layer(_att(2, 1, 128, 128, 0.09, 0, 0.25, 64), _moe(16, 6, 0, 1)),
])

# a width and a vocabulary that are multiples of nothing useful, three heads everywhere, five taps, a latent attention
# without plain query entries is not in the design: the smallest here has two
VAS_D = _model(97, 100, 2e-5, 5, 1000, 1, 0, 8.0, [
    _layer(_lat(3, 2, 10, 14, 18, 9, 0.35, 777.0, 10, _yarn(3.0, 24, 6.0, 0.75)), _moe(12, 7, 1, 3)),
    _layer(_delta(3, 3, 9, 14, 3), _dense(52)),
    _layer(_att(3, 3, 10, 14, 0.3, 11, 2.0, 5), _dense(52)),
])

VAS = {"a": VAS_A, "b": VAS_B, "c": VAS_C, "d": VAS_D}

# for one long request: more than a thousand positions against an `original` length of 128 (every branch of the
# stretch is met), a window that passes over hundreds of decoded tokens, temperatures that step several times,
# decoded tokens whose keys are split over several CTAs, a delta state that lives through all of it
_L_ROT = (100000.0, 32, _yarn(8.0, 128, 32.0, 1.0))
VAS_LONG = _model(500, 256, 1e-6, 3, 4099, 131, 17, 20.0, [
    _layer(_att(8, 2, 64, 32, 0.125, 200, 0.5, 100), _dense(96)),
    _layer(_lat(4, 32, 32, 48, 96, 64, 0.12, *_L_ROT), _moe(32, 8, 2, 2)),
    _layer(_delta(4, 2, 32, 48, 4), _dense(64)),
    _layer(_lat(4, 32, 32, 32, 96, 48, 0.12, *_L_ROT, kv_from=1), None),
])


def tensor_shapes(cfg: dict) -> dict[str, tuple[int, ...]]:
    V, W, taps = cfg["vocab"], cfg["width"], cfg["canon"]["taps"]
    shapes: dict[str, tuple[int, ...]] = {"embed": (V, W), "bigram": (cfg["embedding"]["bigram"]["buckets"] + 1, W), "final.norm": (),
                                          "head": (V, W)}
    for i, layer in enumerate(cfg["layers"]):
        p, m, q = f"l{i}.", layer["mixer"], f"l{i}.mix."
        shapes.update({p + "norm1": (), p + "norm1b": (), p + "canon1": (W, taps)})
        if layer["type"] == "attention":
            H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            shapes.update({q + "q": (H * d, W), q + "k": (G * d, W), q + "v": (G * e, W), q + "r1": (H,), q + "r2": (H,), q + "o": (W, H * e)})
        elif layer["type"] == "latent_attention":
            H, d, r, e, R, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            shapes.update({q + "dq": (Q, W), q + "dq.norm": (Q,), q + "uq": (H * (d + r), Q), q + "uk": (H * d, R), q + "uv": (H * e, R),
                           q + "o": (W, H * e)})
            if m.get("kv_from") is None:
                shapes.update({q + "dkv": (R + r, W), q + "dkv.norm": (R,)})
        else:
            H, G, d, e, K = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            shapes.update({q + "q": (G * d, W), q + "q.conv": (G * d, K), q + "k": (G * d, W), q + "k.conv": (G * d, K), q + "v": (H * e, W),
                           q + "v.conv": (H * e, K), q + "b": (H, W), q + "a": (H, W), q + "A_log": (H,), q + "dt_bias": (H,),
                           q + "g": (H * e, W), q + "norm": (e,), q + "o": (W, H * e)})
        mlp = layer["mlp"]
        if mlp is not None:
            shapes.update({p + "norm2": (), p + "norm2b": (), p + "canon2": (W, taps)})
            f = p + "mlp."
            if mlp["kind"] == "dense":
                shapes.update({f + "gate": (mlp["ff"], W), f + "up": (mlp["ff"], W), f + "down": (W, mlp["ff"])})
            else:
                outputs = mlp["router"]["experts"] + mlp["router"]["identity"]
                shapes.update({f + "router": (outputs, W), f + "correction": (outputs,)})
                for e in range(mlp["router"]["experts"]):
                    shapes.update({f"{f}e{e}.up": (mlp["expert"]["ff"], W), f"{f}e{e}.down": (W, mlp["expert"]["ff"])})
    return shapes


def vasosun_weights(cfg: dict, seed: int, *, sharp: float = 1.0, routed_share: float = 1.0) -> dict[str, torch.Tensor]:
    """Float32 weights whose values are all representable in bfloat16 (a bfloat16 run reads exactly
    what the plain model reads).  Matrices N(0, 1/fan_in), the norms' numbers around one, the
    embedding tables N(0, 1); taps of the convolutions around a half; distance numbers r1 around a
    half (either sign), r2 positive; decay rates and step sizes such that a delta state lives for
    tens of tokens; corrections of a few tenths.  `sharp` multiplies the matrices that make queries
    (a softmax that picks few keys shows one wrong key or a window that is one position off far
    beyond rounding).  `routed_share` multiplies the number of the norm behind every routed
    feed-forward: a router is a step function of its input, so a run in a narrower number format,
    which now and then chooses another expert than the plain model, is compared with a small share."""
    routed = {f"l{i}.norm2b" for i, layer in enumerate(cfg["layers"]) if layer["mlp"] is not None and layer["mlp"]["kind"] == "moe"}
    out: dict[str, torch.Tensor] = {}
    shapes = tensor_shapes(cfg)
    for name, shape in shapes.items():
        x = seeded_normal(shape if shape else (1,), f"vasosun:{seed}:{name}")
        if not shape:
            x = (1.0 + 0.1 * x).reshape(())
            if name in routed:
                x = x * routed_share
        elif name in ("embed", "bigram"):
            pass
        elif name.endswith((".canon1", ".canon2", ".conv")):
            x = 0.5 * x / float(shape[1]) ** 0.5 + (0.3 if name.endswith(".conv") else 0.0)
        elif name.endswith(".r1"):
            x = 0.5 + 0.5 * x
        elif name.endswith(".r2"):
            x = 0.05 + (0.5 + 0.3 * x).abs()
        elif name.endswith("dt_bias"):
            x = -3.0 + 0.7 * x
        elif name.endswith("A_log"):
            x = 0.3 + 0.4 * x
        elif name.endswith(".correction"):
            x = 0.1 * x
        elif len(shape) == 1:
            x = 1.0 + 0.1 * x
        else:
            x = x / float(shape[1]) ** 0.5
            if name.endswith((".mix.uq",)) or (name.endswith(".mix.q") and name[:-1] + "r1" in shapes):
                x = x * sharp
            if name.endswith((".mix.b", ".mix.a", ".mlp.router")):
                x = x * 2.0  # gates and choices that depend on the token
        out[name] = x.to(torch.bfloat16).to(torch.float32)
    return out


def write_vasosun_folder(folder: Path, cfg: dict, weights: dict[str, torch.Tensor], dtype: Optional[torch.dtype] = torch.bfloat16) -> Path:
    """config.json + model.safetensors, written with the safetensors package (not the engine's writer)."""
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    save_file({k: (v if dtype is None else v.to(dtype)).contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))
    return folder


def random_ids(cfg: dict, n: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()
