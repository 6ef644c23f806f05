"""The tests' own small Pekunex configurations and weights (no product code here).

The configurations differ from one another in every size and option: head counts and grouping
(every query head with its own keys, all with one), key widths against value widths (narrower,
equal, wider; multiples of 16 and not), how much of a head turns (nothing, a part, all of it),
both kinds of stretched frequencies with requests longer and shorter than the `original` length,
a score cap or none, the matrix memory's widths and gate cap, the state-space layer's heads,
groups (one per head, one for all), state width, taps (two to five) and norm parts (one included),
layers without a feed-forward, layers that run with another layer's weights, and the constants on
the embedding and the logits (one included).  Weights come from the tests' integer-hash generator
under the checkpoint's tensor names.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Optional

import torch

from tests.tiny_configs import seeded_normal


def _rot(base, dims, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling is not None:
        r["scaling"] = scaling
    return r


def _yarn(factor, original, fast, slow):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


def _llama(factor, low, high, original):
    return {"factor": factor, "low": low, "high": high, "original": original}


def _att(heads, kv_heads, dim, vdim, scale, rot, softcap=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        m["rot"] = rot
    if softcap is not None:
        m["softcap"] = softcap
    return {"type": "attention", "mixer": m}


def _par(left, right, left_scale, right_scale):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}}


def _left(heads, kv_heads, dim, vdim, scale, rot):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        m["rot"] = rot
    return m


def _right(heads, dim, vdim, gate_cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": gate_cap}


def _ssm(heads, vdim, state, groups, conv, norm_groups):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}}


def _layer(mixer, ff, weights_of=None):
    entry = dict(mixer, mlp=None if ff is None else {"kind": "dense", "ff": ff})
    if weights_of is not None:
        entry["weights_of"] = weights_of
    return entry


# all three mixers; values narrower than keys in one attention and wider in the other; a third of a head turns; a layer
# without a feed-forward; the last two layers run with the weights of earlier ones (a state-space layer and an attention)
_A0 = _att(4, 2, 24, 16, 0.9, _rot(10000.0, 8, _yarn(4.0, 32, 8.0, 1.0)), softcap=9.0)
_A1 = _par(_left(3, 1, 16, 20, 0.6, _rot(5000.0, 16, _llama(8.0, 1.0, 4.0, 32))), _right(3, 12, 20, 8.0), 0.7, 1.3)
_A2 = _ssm(4, 12, 8, 2, 3, 4)
PEK_A = {
    "architecture": "Pekunex", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0}, "logit_scale": 0.5,
    "layers": [_layer(_A0, 40), _layer(_A1, None), _layer(_A2, 56), _layer(_A2, 56, weights_of=2), _layer(_A0, 40, weights_of=0)],
}

# the recurrent mixers alone: one head with odd widths and one group, one norm part, two taps; a group per head and five
# taps; a matrix memory with one head and keys wider than values; constants of one on the embedding and the logits
PEK_B = {
    "architecture": "Pekunex", "vocab": 130, "width": 72, "norm": {"eps": 3e-6}, "embedding": {"scale": 1.0}, "logit_scale": 1.0,
    "layers": [
        _layer(_ssm(1, 7, 5, 1, 2, 1), 20),
        _layer(_par(_left(2, 2, 10, 6, 0.4, None), _right(1, 11, 6, 3.0), 1.0, 1.0), 36),
        _layer(_ssm(6, 10, 20, 6, 5, 3), None),
        _layer(_par(_left(4, 1, 8, 8, 0.5, _rot(300.0, 4)), _right(5, 6, 9, 20.0), -0.5, 2.0), 24),
    ],
}

# attention alone: every query head with its own keys, or all with one; whole heads turn, or nothing; no cap on one
# layer; plain frequencies on another; the first layer's weights run again at the end
_C0 = _att(6, 6, 16, 16, 1.2, _rot(500.0, 16, _yarn(2.0, 48, 4.0, 0.5)), softcap=5.0)
PEK_C = {
    "architecture": "Pekunex", "vocab": 300, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.5}, "logit_scale": 2.0,
    "layers": [
        _layer(_C0, 32),
        _layer(_att(5, 1, 12, 28, 1.5, None, softcap=50.0), None),
        _layer(_att(2, 2, 64, 32, 0.5, _rot(123456.0, 32)), 48),
        _layer(_C0, 32, weights_of=0),
    ],
}

# heads of 128 and of 64 (the widths the tensor-core attention kernels take), one key/value head for both query heads;
# recurrent layers as wide, a state of 64 channels
PEK_D = {
    "architecture": "Pekunex", "vocab": 180, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 2.0}, "logit_scale": 0.25,
    "layers": [
        _layer(_att(2, 1, 128, 128, 0.7, _rot(1000000.0, 64, _yarn(8.0, 64, 16.0, 2.0)), softcap=20.0), 64),
        _layer(_par(_left(4, 2, 64, 64, 0.25, _rot(10000.0, 64, _llama(4.0, 1.0, 2.0, 40))), _right(2, 64, 64, 15.0), 1.5, 0.5), 64),
        _layer(_ssm(2, 64, 64, 1, 4, 2), None),
        _layer(_att(4, 4, 64, 48, 0.8, _rot(10000.0, 16), softcap=30.0), 96),
    ],
}

# for one long request: more than a thousand positions against `original` lengths of 256 and 128 (every branch of both
# stretches is met), decoded tokens whose keys are split over several CTAs, the recurrences in segments side by side
PEK_LONG = {
    "architecture": "Pekunex", "vocab": 500, "width": 256, "norm": {"eps": 1e-6}, "embedding": {"scale": 4.0}, "logit_scale": 0.5,
    "layers": [
        _layer(_att(8, 2, 128, 64, 1.0, _rot(100000.0, 96, _yarn(4.0, 256, 32.0, 1.0)), softcap=25.0), 96),
        _layer(_par(_left(4, 4, 64, 64, 0.4, _rot(50000.0, 64, _llama(8.0, 1.0, 4.0, 128))), _right(4, 32, 48, 10.0), 1.1, 0.6), 96),
        _layer(_ssm(8, 32, 16, 2, 4, 2), 64),
        _layer(_ssm(8, 32, 16, 2, 4, 2), 64, weights_of=2),
    ],
}

# a width and a vocabulary that are multiples of nothing useful, three heads everywhere; the layers begin with the
# state-space mixer, and it is the pair side by side whose weights run a second time
_E1 = _par(_left(2, 1, 12, 10, 0.5, _rot(777.0, 12, _llama(3.0, 0.5, 2.0, 50))), _right(3, 16, 12, 6.0), 0.9, 1.1)
PEK_E = {
    "architecture": "Pekunex", "vocab": 97, "width": 100, "norm": {"eps": 2e-5}, "embedding": {"scale": 1.7}, "logit_scale": 1.3,
    "layers": [
        _layer(_ssm(3, 9, 6, 3, 3, 3), 52),
        _layer(_E1, 52),
        _layer(_att(3, 3, 10, 14, 1.1, _rot(2000.0, 6, _yarn(3.0, 24, 6.0, 0.75)), softcap=12.0), None),
        _layer(_E1, 52, weights_of=1),
    ],
}

PEK = {"a": PEK_A, "b": PEK_B, "c": PEK_C, "d": PEK_D, "e": PEK_E}


def _attention_shapes(p: str, m: dict, W: int, biased: bool) -> dict[str, tuple[int, ...]]:
    nq, nk, nv, no = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"], m["heads"] * m["vdim"]
    shapes = {p + "q": (nq, W), p + "k": (nk, W), p + "v": (nv, W), p + "o": (W, no)}
    if biased:
        shapes.update({p + "q.b": (nq,), p + "k.b": (nk,), p + "v.b": (nv,), p + "g": (no, W)})
    else:
        shapes[p + "sink"] = (m["heads"],)
    return shapes


def tensor_shapes(cfg: dict) -> dict[str, tuple[int, ...]]:
    V, W = cfg["vocab"], cfg["width"]
    shapes: dict[str, tuple[int, ...]] = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for i, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p, m = f"l{i}.", layer["mixer"]
        shapes.update({p + "norm1": (W,), p + "norm2": (W,)})
        if layer["type"] == "attention":
            shapes.update(_attention_shapes(p + "mix.", m, W, True))
        elif layer["type"] == "parallel":
            shapes.update(_attention_shapes(p + "mix.left.", m["left"], W, False))
            r, q = m["right"], p + "mix.right."
            hd, he = r["heads"] * r["dim"], r["heads"] * r["vdim"]
            shapes.update({q + "q": (hd, W), q + "k": (hd, W), q + "v": (he, W), q + "g": (he, W), q + "o": (W, he), q + "norm": (he,),
                           q + "i": (r["heads"], W), q + "i.b": (r["heads"],), q + "f": (r["heads"], W), q + "f.b": (r["heads"],)})
        else:
            inner, gn, H = m["heads"] * m["vdim"], m["groups"] * m["state"], m["heads"]
            q = p + "mix."
            shapes.update({q + "in": (2 * inner + 2 * gn + H, W), q + "conv": (inner + 2 * gn, m["conv"]), q + "conv.b": (inner + 2 * gn,),
                           q + "dt_bias": (H,), q + "A_log": (H,), q + "D": (H,), q + "norm": (inner,), q + "o": (W, inner)})
        if layer["mlp"]:
            ff = layer["mlp"]["ff"]
            shapes.update({p + "mlp.gate": (ff, W), p + "mlp.up": (ff, W), p + "mlp.down": (W, ff)})
    return shapes


def pekunex_weights(cfg: dict, seed: int, *, sharp: float = 1.0) -> dict[str, torch.Tensor]:
    """Float32 weights whose values are all representable in bfloat16 (a bfloat16 run reads exactly
    what the plain model reads).  Matrices N(0, 1/fan_in), norm weights around one, biases and
    sinks around zero, the embedding N(0, 1); forget-gate biases around three and step sizes around
    a tenth, so that memories and states live for tens of tokens; decay rates between one and a
    few.  `sharp` multiplies the query matrices of the attention with sinks and of the matrix
    memory (the capped attention's scores are sharpened through its configured scale, since its
    queries are brought to unit size): a softmax that picks few keys shows one wrong key, an edge
    that is one position off or a lost sink far beyond rounding."""
    out: dict[str, torch.Tensor] = {}
    for name, shape in tensor_shapes(cfg).items():
        x = seeded_normal(shape, f"pekunex:{seed}:{name}")
        if name == "embed":
            pass
        elif name.endswith(".f.b"):
            x = 3.0 + x
        elif name.endswith("dt_bias"):
            x = -2.0 + 0.7 * x
        elif name.endswith("A_log"):
            x = 0.5 + 0.5 * x
        elif name.endswith((".D", ".sink")):
            x = 0.5 * x + (1.0 if name.endswith(".D") else 0.0)
        elif name.endswith((".b", ".i.b")):
            x = 0.3 * x
        elif name.endswith(".conv"):
            x = x / float(shape[1]) ** 0.5
        elif len(shape) == 1:
            x = 1.0 + 0.1 * x
        else:
            x = x / float(shape[1]) ** 0.5
            if name.endswith((".left.q", ".right.q")):
                x = x * sharp
            if name.endswith((".i", ".f")):
                x = x * 2.0  # gates that depend on the token
        out[name] = x.to(torch.bfloat16).to(torch.float32)
    return out


def write_pekunex_folder(folder: Path, cfg: dict, weights: dict[str, torch.Tensor], dtype: Optional[torch.dtype] = torch.bfloat16) -> Path:
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
