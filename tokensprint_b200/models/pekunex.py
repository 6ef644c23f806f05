"""Pekunex: its typed configuration and the architecture entry.

A decoder of pre-normed layers (x <- x + mixer(norm1(x)); x <- x + ff(norm2(x)) where the layer has
a feed-forward).  A layer's mixer is one of three.  "attention": grouped-query softmax attention with
biased projections, a rotation whose frequencies are stretched by a ramp between two wavelengths and
whose cosines and sines carry a magnitude, q and k divided by their root mean square after the
rotation, scores bent through a tanh cap, and a sigmoid gate on the concatenated heads.  "parallel":
two mixers on the same input whose outputs are added with fixed weights: a softmax attention with a
learned sink per head and piecewise stretched frequencies, beside a matrix memory with exponential
gates that a running maximum keeps in range.  "mamba2": a selective state-space recurrence with a
scalar decay per head, a short causal convolution on its inputs, and a gate and a norm in groups on
the way out.  A layer may use another layer's weights with a cache and state of its own.  Embedding
rows and logits are multiplied by constants.  Every size and every constant that may differ between
two models of the design comes from config.json:

    architecture, vocab, width, norm.eps, embedding.scale, logit_scale
    layers[i] {type, mixer {...}, mlp null | {kind: "dense", ff}, weights_of (optional)}
      type "attention": mixer {heads, kv_heads, dim, vdim, scale, softcap (optional),
                               rot {base, dims, scaling {factor, original, fast, slow} (optional)} (optional)}
      type "parallel":  mixer {left_scale, right_scale,
                               left {heads, kv_heads, dim, vdim, scale,
                                     rot {base, dims, scaling {factor, low, high, original} (optional)} (optional)},
                               right {heads, dim, vdim, gate_cap}}
      type "mamba2":    mixer {heads, vdim, state, groups, conv, norm_groups}

Tensor names: embed, l<i>.norm1/.norm2, l<i>.mix.{q,q.b,k,k.b,v,v.b,g,o},
l<i>.mix.left.{q,k,v,sink,o}, l<i>.mix.right.{q,k,v,g,o,norm,i,i.b,f,f.b},
l<i>.mix.{in,conv,conv.b,dt_bias,A_log,D,norm,o}, l<i>.mlp.{gate,up,down}, final.norm, head.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Optional, Union

from tokensprint_b200.config.model_config import ConfigError, read_config_json, require, write_config_json
from tokensprint_b200.config.registry import PRESET_DIR, register_architecture, register_preset
from tokensprint_b200.models.spec import ModelSpec, RunSpec
from tokensprint_b200.parts.base import PartSpec

ARCHITECTURE = "Pekunex"
DEFAULT_MAX_POSITIONS = 32768  # the design sets no limit; what the engine plans for unless the file says otherwise


def _section(d: dict[str, Any], key: str, where: str) -> dict[str, Any]:
    value = d.get(key)
    if not isinstance(value, dict):
        raise ConfigError(f"config.json: {where}'{key}' must be an object")
    return value


@dataclass(frozen=True)
class RotationConfig:
    """Rotate-half rotation of the first `dims` entries of a head; `scaling` holds the stretch's
    numbers with `kind` "yarn" or "llama3" added (None: plain frequencies)."""

    base: float
    dims: int
    scaling: Optional[tuple[tuple[str, Any], ...]] = None

    @classmethod
    def from_dict(cls, d: Optional[dict[str, Any]], kind: str, keys: tuple[str, ...], dim: int, where: str) -> Optional["RotationConfig"]:
        if d is None:
            return None
        scaling = d.get("scaling")
        if scaling is not None:
            scaling = tuple([("kind", kind)] + [(k, require(scaling, k, float)) for k in keys])
        c = cls(base=require(d, "base", float), dims=require(d, "dims", int), scaling=scaling)
        if c.dims % 2 or not 0 <= c.dims <= dim or c.base <= 1.0:
            raise ConfigError(f"config.json: {where}rot.dims must be even and at most dim, rot.base above 1")
        return c

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            d["scaling"] = {k: v for k, v in self.scaling if k != "kind"}
        return d

    def part(self) -> Optional[PartSpec]:
        if self.dims == 0:
            return None
        return PartSpec("rotary", {"dim": self.dims, "theta": self.base, "exact_frequencies": True,
                                   "scaling": None if self.scaling is None else dict(self.scaling)})


def _heads(d: dict[str, Any], where: str) -> tuple[int, int, int, int, float]:
    heads, kv_heads, dim, vdim = (require(d, k, int) for k in ("heads", "kv_heads", "dim", "vdim"))
    if min(heads, kv_heads, dim, vdim) < 1 or heads % kv_heads:
        raise ConfigError(f"config.json: {where}heads must be a positive multiple of kv_heads, dim and vdim positive")
    return heads, kv_heads, dim, vdim, require(d, "scale", float)


@dataclass(frozen=True)
class CappedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float  # 0: the scores are not bent
    rot: Optional[RotationConfig]

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "CappedAttentionConfig":
        heads, kv_heads, dim, vdim, scale = _heads(d, where)
        softcap = require(d, "softcap", float) if d.get("softcap") is not None else 0.0
        if softcap < 0:
            raise ConfigError(f"config.json: {where}softcap must be positive")
        return cls(heads, kv_heads, dim, vdim, scale, softcap,
                   RotationConfig.from_dict(d.get("rot"), "yarn", ("factor", "original", "fast", "slow"), dim, where))

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.softcap:
            d["softcap"] = self.softcap
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d

    def part(self, width: int, eps: float, p: str) -> PartSpec:
        return PartSpec("attention", {
            "hidden_size": width, "num_heads": self.heads, "num_kv_heads": self.kv_heads, "head_dim": self.dim, "value_dim": self.vdim,
            "scale": self.scale, "softcap": self.softcap, "qk_norm": "unit_after_rotation", "qk_norm_eps": eps,
            "position": None if self.rot is None else self.rot.part(),
            "q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o", "gate": p + "g", "q_bias": p + "q.b", "k_bias": p + "k.b", "v_bias": p + "v.b"})


@dataclass(frozen=True)
class SinkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[RotationConfig]

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "SinkAttentionConfig":
        heads, kv_heads, dim, vdim, scale = _heads(d, where)
        return cls(heads, kv_heads, dim, vdim, scale,
                   RotationConfig.from_dict(d.get("rot"), "llama3", ("factor", "low", "high", "original"), dim, where))

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d

    def part(self, width: int, p: str) -> PartSpec:
        return PartSpec("attention", {
            "hidden_size": width, "num_heads": self.heads, "num_kv_heads": self.kv_heads, "head_dim": self.dim, "value_dim": self.vdim,
            "scale": self.scale, "position": None if self.rot is None else self.rot.part(), "sinks": p + "sink",
            "q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o"})


@dataclass(frozen=True)
class MatrixMemoryConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "MatrixMemoryConfig":
        c = cls(require(d, "heads", int), require(d, "dim", int), require(d, "vdim", int), require(d, "gate_cap", float))
        if min(c.heads, c.dim, c.vdim) < 1 or not c.gate_cap > 0:
            raise ConfigError(f"config.json: {where}heads, dim, vdim and gate_cap must be positive")
        return c

    def to_dict(self) -> dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "gate_cap": self.gate_cap}

    def part(self, width: int, eps: float, p: str) -> PartSpec:
        return PartSpec("matrix_memory", {
            "hidden_size": width, "num_heads": self.heads, "key_dim": self.dim, "value_dim": self.vdim, "gate_cap": self.gate_cap,
            "norm_eps": eps, "q": p + "q", "k": p + "k", "v": p + "v", "gate": p + "g", "o": p + "o", "norm": p + "norm",
            "input_gate": p + "i", "input_gate_bias": p + "i.b", "forget_gate": p + "f", "forget_gate_bias": p + "f.b"})


@dataclass(frozen=True)
class SideBySideConfig:
    left: SinkAttentionConfig
    right: MatrixMemoryConfig
    left_scale: float
    right_scale: float

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "SideBySideConfig":
        return cls(SinkAttentionConfig.from_dict(_section(d, "left", where), where + "left."),
                   MatrixMemoryConfig.from_dict(_section(d, "right", where), where + "right."),
                   require(d, "left_scale", float), require(d, "right_scale", float))

    def to_dict(self) -> dict[str, Any]:
        return {"left": self.left.to_dict(), "right": self.right.to_dict(), "left_scale": self.left_scale, "right_scale": self.right_scale}

    def part(self, width: int, eps: float, p: str) -> PartSpec:
        return PartSpec("parallel", {"mixers": [self.left.part(width, p + "left."), self.right.part(width, eps, p + "right.")],
                                     "scales": [self.left_scale, self.right_scale]})


@dataclass(frozen=True)
class StateSpaceConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "StateSpaceConfig":
        c = cls(*(require(d, k, int) for k in ("heads", "vdim", "state", "groups", "conv", "norm_groups")))
        if min(c.heads, c.vdim, c.state, c.groups, c.conv, c.norm_groups) < 1 or c.heads % c.groups or (c.heads * c.vdim) % c.norm_groups:
            raise ConfigError(f"config.json: {where}sizes must be positive, heads a multiple of groups, heads * vdim of norm_groups")
        return c

    def to_dict(self) -> dict[str, Any]:
        return {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups, "conv": self.conv,
                "norm_groups": self.norm_groups}

    def part(self, width: int, eps: float, p: str) -> PartSpec:
        return PartSpec("state_space", {
            "hidden_size": width, "num_heads": self.heads, "value_dim": self.vdim, "state_dim": self.state, "groups": self.groups,
            "taps": self.conv, "norm_groups": self.norm_groups, "norm_eps": eps, "in_proj": p + "in", "conv": p + "conv",
            "conv_bias": p + "conv.b", "dt_bias": p + "dt_bias", "a_log": p + "A_log", "skip": p + "D", "norm": p + "norm", "o": p + "o"})


MIXER_CONFIGS = {"attention": CappedAttentionConfig, "parallel": SideBySideConfig, "mamba2": StateSpaceConfig}
MixerConfig = Union[CappedAttentionConfig, SideBySideConfig, StateSpaceConfig]


@dataclass(frozen=True)
class PekunexLayerConfig:
    type: str
    mixer: MixerConfig
    ff: int = 0  # 0: the layer has no feed-forward
    weights_of: Optional[int] = None  # the layer whose tensors this one uses (None: its own)


@dataclass(frozen=True)
class PekunexConfig:
    """All sizes and constants of one Pekunex model."""

    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_scale: float
    layers: tuple[PekunexLayerConfig, ...]
    max_position_embeddings: int = DEFAULT_MAX_POSITIONS
    eos_token_id: int = -1
    extra: dict[str, Any] = field(default_factory=dict, compare=False, repr=False)

    def __post_init__(self) -> None:
        if self.vocab < 1 or self.width < 1 or not self.layers:
            raise ConfigError("config.json: 'vocab', 'width' and the number of layers must be positive")
        if self.norm_eps <= 0:
            raise ConfigError("config.json: 'norm.eps' must be positive")
        for i, layer in enumerate(self.layers):
            j = layer.weights_of
            if j is not None:
                if not 0 <= j < len(self.layers) or j == i or self.layers[j].weights_of is not None:
                    raise ConfigError(f"config.json: layers[{i}].weights_of must name another layer that has tensors of its own")
                other = self.layers[j]
                if (other.type, other.mixer, other.ff) != (layer.type, layer.mixer, layer.ff):
                    raise ConfigError(f"config.json: layers[{i}] uses the weights of layers[{j}] but describes another layer")

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    def weight_owner(self, i: int) -> int:
        j = self.layers[i].weights_of
        return i if j is None else j

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "PekunexConfig":
        entries = d.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a list with an entry per layer")
        layers = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]."
            kind = entry.get("type")
            if kind not in MIXER_CONFIGS:
                raise ConfigError(f"config.json: {where}type {kind!r} is no mixer of this design (known: {sorted(MIXER_CONFIGS)})")
            mlp = entry.get("mlp")
            if mlp is not None and mlp.get("kind") != "dense":
                raise ConfigError(f"config.json: {where}mlp.kind must be 'dense', got {mlp.get('kind')!r}")
            ff = 0 if mlp is None else require(mlp, "ff", int)
            if mlp is not None and ff < 1:
                raise ConfigError(f"config.json: {where}mlp.ff must be positive")
            owner = entry.get("weights_of")
            layers.append(PekunexLayerConfig(type=kind, mixer=MIXER_CONFIGS[kind].from_dict(_section(entry, "mixer", where), where), ff=ff,
                                             weights_of=None if owner is None else int(owner)))
        known = {"architecture", "architectures", "model_type", "vocab", "width", "norm", "layers", "embedding", "logit_scale",
                 "max_position_embeddings", "eos_token_id"}
        return cls(
            vocab=require(d, "vocab", int), width=require(d, "width", int), norm_eps=require(_section(d, "norm", ""), "eps", float),
            embedding_scale=require(d["embedding"], "scale", float) if isinstance(d.get("embedding"), dict) else 1.0,
            logit_scale=require(d, "logit_scale", float) if d.get("logit_scale") is not None else 1.0, layers=tuple(layers),
            max_position_embeddings=int(d.get("max_position_embeddings") or DEFAULT_MAX_POSITIONS),
            eos_token_id=int(d["eos_token_id"]) if isinstance(d.get("eos_token_id"), int) else -1,
            extra={k: v for k, v in d.items() if k not in known})

    @classmethod
    def from_json(cls, path: str | Path) -> "PekunexConfig":
        return cls.from_dict(read_config_json(path))

    def to_dict(self) -> dict[str, Any]:
        layers = []
        for l in self.layers:
            entry: dict[str, Any] = {"type": l.type, "mixer": l.mixer.to_dict(), "mlp": None if not l.ff else {"kind": "dense", "ff": l.ff}}
            if l.weights_of is not None:
                entry["weights_of"] = l.weights_of
            layers.append(entry)
        d: dict[str, Any] = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                             "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale, "layers": layers}
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            d["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_id >= 0:
            d["eos_token_id"] = self.eos_token_id
        return d

    def save(self, folder: str | Path) -> None:
        write_config_json(folder, self.to_dict())


@register_architecture(ARCHITECTURE, model_types=("pekunex",), config_from_dict=PekunexConfig.from_dict)
def build_pekunex_spec(config: PekunexConfig) -> ModelSpec:
    W, eps = config.width, config.norm_eps

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"dim": W, "eps": eps, "weight": name})

    blocks: list[PartSpec] = []  # one per layer that has tensors of its own
    block_of: dict[int, int] = {}
    ignorable: list[str] = []
    for i, layer in enumerate(config.layers):
        if layer.weights_of is not None:
            continue
        p = f"l{i}."
        m = layer.mixer
        mixer = m.part(W, eps, p + "mix.")
        params: dict[str, Any] = {"mixer": mixer, "mixer_norm": norm(p + "norm1")}
        if layer.ff:
            params.update(ffn_norm=norm(p + "norm2"), feed_forward=PartSpec("swiglu", {
                "hidden_size": W, "intermediate_size": layer.ff, "gate": p + "mlp.gate", "up": p + "mlp.up", "down": p + "mlp.down"}))
        else:
            ignorable.append(p + "norm2")  # a layer without a feed-forward has no use for it
        block_of[i] = len(blocks)
        blocks.append(PartSpec("pre_norm", params))
    # a layer that names another's weights is a second run of that layer's block, with a cache and state of its own
    runs = [RunSpec(layer=block_of[config.weight_owner(i)]) for i in range(len(config.layers))]
    return ModelSpec(
        vocab_size=config.vocab, hidden_size=W, embedding="embed", layers=blocks, final_norm=norm("final.norm"), lm_head="head",
        run_order=runs, embedding_scale=config.embedding_scale, max_positions=config.max_position_embeddings,
        eos_token_id=config.eos_token_id, ignorable_tensors=tuple(ignorable),
        logits_transform=None if config.logit_scale == 1.0 else PartSpec("scale", {"factor": config.logit_scale}))


# Named models of this design, so that the command lines can run them with random weights.
for _path in sorted(PRESET_DIR.glob("pekunex-*.json")):
    register_preset("pekunex", _path.stem, _path)
