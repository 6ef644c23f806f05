"""Vasosun: its typed configuration and the architecture entry.

A decoder whose sublayers stand between two norms of one learned number each and read their normed
input h as h + conv(h), a short causal convolution over time on every channel:

    x <- x + norm1b(mixer(h1 + conv1(h1))),  h1 = norm1(x)
    x <- x + norm2b(ff(h2 + conv2(h2))),     h2 = norm2(x)       (where the layer has a feed-forward)

A layer's mixer is one of three.  "attention": grouped-query softmax attention over a sliding
window, without a rotation; the queries at position p are multiplied by 1 + coef ln(floor((p + 1) /
every) + 1), and the scaled score of key j for query i loses r1_h ln(1 + r2_h (i - j)) with two
learned numbers per head.  "latent_attention": causal attention whose queries pass a normed latent
and whose keys and values are rebuilt from a normed latent c plus one rotated key part for all
heads (neighbouring entries turn together; frequencies stretched by a ramp between two wavelengths,
cosines and sines times 0.1 ln(factor) + 1); only [c ; rotated part] is cached, and a layer may read
the rows another layer cached (`kv_from`) with matrices of its own.  "delta": the gated delta rule
(short convolutions and silu on q, k, v, unit q and k, a write strength and a decay per head, a norm
per head with a silu gate).  The feed-forward is a dense SwiGLU or a set of routed experts
W_down gelu(W_up h) chosen by softmax scores plus a correction, whose weights are the scores
themselves and whose last router outputs are identity experts.  The embedding adds a row of a table
hashed from the token before and the token; the logits pass cap * tanh(logits / cap).  Every size and
every constant that may differ between two models of the design comes from config.json:

    architecture, vocab, width, norm.eps, canon.taps, embedding.bigram {buckets, mul_prev, mul_cur}, logit_softcap
    layers[i] {type, mixer {...}, mlp null | {kind: "dense", ff} | {kind: "moe", expert {ff}, router {experts, identity, top}}}
      type "attention":        mixer {heads, kv_heads, dim, vdim, scale, mask {size}, q_temp {coef, every}}
      type "latent_attention": mixer {heads, dim, rot_dim, vdim, kv_rank, q_rank, scale,
                                      rot {base, dims, scaling {factor, original, fast, slow} (optional)}, kv_from (optional)}
      type "delta":            mixer {heads, kv_heads, dim, vdim, conv}

Tensor names: embed, bigram, l<i>.norm1/.norm1b/.norm2/.norm2b (one number each), l<i>.canon1/.canon2,
l<i>.mix.{q,k,v,r1,r2,o}, l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,o},
l<i>.mix.{q,q.conv,k,k.conv,v,v.conv,b,a,A_log,dt_bias,g,norm,o}, l<i>.mlp.{gate,up,down},
l<i>.mlp.{router,correction,e<j>.up,e<j>.down}, final.norm, head.
Constants in code are those the design fixes: 1e-6 under the unit length of q and k and the key
width's inverse root on q in the delta rule, 0.1 ln(factor) + 1 and 0.001 in the stretched rotation.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Optional, Union

from tokensprint_b200.config.model_config import ConfigError, read_config_json, require, write_config_json
from tokensprint_b200.config.registry import PRESET_DIR, register_architecture, register_preset
from tokensprint_b200.models.spec import ModelSpec, RunSpec
from tokensprint_b200.parts.base import PartSpec

ARCHITECTURE = "Vasosun"
DEFAULT_MAX_POSITIONS = 32768  # the design sets no limit; what the engine plans for unless the file says otherwise


def _section(d: dict[str, Any], key: str, where: str) -> dict[str, Any]:
    value = d.get(key)
    if not isinstance(value, dict):
        raise ConfigError(f"config.json: {where}'{key}' must be an object")
    return value


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int        # 0: every earlier key
    temp_coef: float
    temp_every: int    # 0: no query temperature

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "WindowAttentionConfig":
        heads, kv_heads, dim, vdim = (require(d, k, int) for k in ("heads", "kv_heads", "dim", "vdim"))
        if min(heads, kv_heads, dim, vdim) < 1 or heads % kv_heads:
            raise ConfigError(f"config.json: {where}heads must be a positive multiple of kv_heads, dim and vdim positive")
        window = require(_section(d, "mask", where), "size", int) if d.get("mask") is not None else 0
        temp = d.get("q_temp")
        coef, every = (require(temp, "coef", float), require(temp, "every", int)) if temp is not None else (0.0, 0)
        if window < 0 or (temp is not None and every < 1):
            raise ConfigError(f"config.json: {where}mask.size must not be negative and q_temp.every must be positive")
        return cls(heads, kv_heads, dim, vdim, require(d, "scale", float), window, coef, every)

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.window:
            d["mask"] = {"size": self.window}
        if self.temp_every:
            d["q_temp"] = {"coef": self.temp_coef, "every": self.temp_every}
        return d

    def part(self, width: int, eps: float, p: str) -> PartSpec:
        return PartSpec("attention", {
            "hidden_size": width, "num_heads": self.heads, "num_kv_heads": self.kv_heads, "head_dim": self.dim, "value_dim": self.vdim,
            "scale": self.scale, "window": self.window, "distance": (p + "r1", p + "r2"),
            "q_temperature": (self.temp_coef, self.temp_every) if self.temp_every else None,
            "q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o"})


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    rot_scaling: Optional[tuple[tuple[str, float], ...]]  # (factor, original, fast, slow) by name, or None
    kv_from: Optional[int] = None

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "LatentAttentionConfig":
        heads, dim, rot_dim, vdim, kv_rank, q_rank = (require(d, k, int) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"))
        if min(heads, vdim, kv_rank, q_rank) < 1 or dim < 0 or rot_dim < 0 or dim + rot_dim < 1:
            raise ConfigError(f"config.json: {where}heads, vdim, kv_rank and q_rank must be positive, dim + rot_dim too")
        rot = _section(d, "rot", where)
        base, dims = require(rot, "base", float), require(rot, "dims", int)
        if dims % 2 or not 0 <= dims <= rot_dim or base <= 1.0:
            raise ConfigError(f"config.json: {where}rot.dims must be even and at most rot_dim, rot.base above 1")
        scaling = rot.get("scaling")
        if scaling is not None:
            scaling = tuple((k, require(scaling, k, float)) for k in ("factor", "original", "fast", "slow"))
        source = d.get("kv_from")
        return cls(heads, dim, rot_dim, vdim, kv_rank, q_rank, require(d, "scale", float), base, dims, scaling,
                   None if source is None else require(d, "kv_from", int))

    def to_dict(self) -> dict[str, Any]:
        rot: dict[str, Any] = {"base": self.rot_base, "dims": self.rot_dims}
        if self.rot_scaling is not None:
            rot["scaling"] = dict(self.rot_scaling)
        d: dict[str, Any] = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
                             "q_rank": self.q_rank, "scale": self.scale, "rot": rot}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d

    def cached_like(self, other: "LatentAttentionConfig") -> bool:
        """Whether this layer can read the rows `other` caches: same latent width, rotated part and rotation."""
        return (self.kv_rank, self.rot_dim, self.rot_base, self.rot_dims, self.rot_scaling) == (
            other.kv_rank, other.rot_dim, other.rot_base, other.rot_dims, other.rot_scaling)

    def part(self, width: int, eps: float, p: str) -> PartSpec:
        position = None
        if self.rot_dims:
            scaling = None if self.rot_scaling is None else dict(self.rot_scaling, kind="yarn")
            position = PartSpec("rotary", {"dim": self.rot_dims, "theta": self.rot_base, "pairing": "neighbours", "exact_frequencies": True,
                                           "scaling": scaling})
        own = self.kv_from is None
        return PartSpec("latent_attention", {
            "hidden_size": width, "num_heads": self.heads, "nope_dim": self.dim, "rot_dim": self.rot_dim, "value_dim": self.vdim,
            "kv_rank": self.kv_rank, "scale": self.scale, "norm_eps": eps, "position": position, "q_rank": self.q_rank,
            "dq": p + "dq", "dq_norm": p + "dq.norm", "q": p + "uq", "dkv": p + "dkv" if own else None,
            "dkv_norm": p + "dkv.norm" if own else None, "uk": p + "uk", "uv": p + "uv", "o": p + "o"})


@dataclass(frozen=True)
class DeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "DeltaConfig":
        c = cls(*(require(d, k, int) for k in ("heads", "kv_heads", "dim", "vdim", "conv")))
        if min(c.heads, c.kv_heads, c.dim, c.vdim, c.conv) < 1 or c.heads % c.kv_heads:
            raise ConfigError(f"config.json: {where}sizes must be positive and heads a multiple of kv_heads")
        return c

    def to_dict(self) -> dict[str, Any]:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}

    def part(self, width: int, eps: float, p: str) -> PartSpec:
        return PartSpec("gated_delta_rule", {
            "hidden_size": width, "num_heads": self.heads, "num_qk_heads": self.kv_heads, "key_dim": self.dim, "value_dim": self.vdim,
            "taps": self.conv, "norm_eps": eps, "unit_eps": 1e-6, "q": p + "q", "k": p + "k", "v": p + "v", "q_conv": p + "q.conv",
            "k_conv": p + "k.conv", "v_conv": p + "v.conv", "beta": p + "b", "decay": p + "a", "a_log": p + "A_log", "dt_bias": p + "dt_bias",
            "gate": p + "g", "norm": p + "norm", "o": p + "o"})


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str          # "dense" or "moe"
    ff: int            # inner width (of every expert, for "moe")
    experts: int = 0
    identity: int = 0
    top: int = 0

    @classmethod
    def from_dict(cls, d: dict[str, Any], where: str) -> "FeedForwardConfig":
        kind = d.get("kind")
        if kind == "dense":
            c = cls("dense", require(d, "ff", int))
        elif kind == "moe":
            router = _section(d, "router", where + "mlp.")
            c = cls("moe", require(_section(d, "expert", where + "mlp."), "ff", int), require(router, "experts", int),
                    require(router, "identity", int) if router.get("identity") is not None else 0, require(router, "top", int))
            if c.experts < 1 or c.identity < 0 or not 0 < c.top <= c.experts + c.identity:
                raise ConfigError(f"config.json: {where}mlp.router: experts positive, identity not negative, top between 1 and their sum")
        else:
            raise ConfigError(f"config.json: {where}mlp.kind must be 'dense' or 'moe', got {kind!r}")
        if c.ff < 1:
            raise ConfigError(f"config.json: {where}mlp: the inner width must be positive")
        return c

    def to_dict(self) -> dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        return {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "identity": self.identity, "top": self.top}}

    def part(self, width: int, p: str) -> PartSpec:
        if self.kind == "dense":
            return PartSpec("swiglu", {"hidden_size": width, "intermediate_size": self.ff, "gate": p + "gate", "up": p + "up", "down": p + "down"})
        return PartSpec("routed_experts", {
            "hidden_size": width, "num_experts": self.experts, "top": self.top, "intermediate_size": self.ff, "router": p + "router",
            "expert_prefix": p + "e", "score": "softmax_all", "correction": p + "correction", "identity": self.identity,
            "activation": "gelu", "weight_on": "output"})


MIXER_CONFIGS = {"attention": WindowAttentionConfig, "latent_attention": LatentAttentionConfig, "delta": DeltaConfig}
MixerConfig = Union[WindowAttentionConfig, LatentAttentionConfig, DeltaConfig]


@dataclass(frozen=True)
class VasosunLayerConfig:
    type: str
    mixer: MixerConfig
    mlp: Optional[FeedForwardConfig] = None


@dataclass(frozen=True)
class VasosunConfig:
    """All sizes and constants of one Vasosun model."""

    vocab: int
    width: int
    norm_eps: float
    canon_taps: int
    bigram_buckets: int
    bigram_mul_prev: int
    bigram_mul_cur: int
    logit_softcap: float
    layers: tuple[VasosunLayerConfig, ...]
    max_position_embeddings: int = DEFAULT_MAX_POSITIONS
    eos_token_id: int = -1
    extra: dict[str, Any] = field(default_factory=dict, compare=False, repr=False)

    def __post_init__(self) -> None:
        if self.vocab < 1 or self.width < 1 or not self.layers:
            raise ConfigError("config.json: 'vocab', 'width' and the number of layers must be positive")
        if self.norm_eps <= 0 or self.canon_taps < 1 or not self.logit_softcap > 0:
            raise ConfigError("config.json: 'norm.eps', 'canon.taps' and 'logit_softcap' must be positive")
        if self.bigram_buckets < 1 or self.bigram_mul_prev < 0 or self.bigram_mul_cur < 0:
            raise ConfigError("config.json: 'embedding.bigram': buckets positive, multipliers not negative")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if isinstance(m, LatentAttentionConfig) and m.kv_from is not None:
                j = m.kv_from
                source = self.layers[j].mixer if 0 <= j < i else None
                if not isinstance(source, LatentAttentionConfig) or source.kv_from is not None or not m.cached_like(source):
                    raise ConfigError(f"config.json: layers[{i}].mixer.kv_from must name an earlier latent attention layer with a latent "
                                      f"of its own and the same kv_rank, rot_dim and rotation")

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "VasosunConfig":
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
            layers.append(VasosunLayerConfig(type=kind, mixer=MIXER_CONFIGS[kind].from_dict(_section(entry, "mixer", where), where),
                                             mlp=None if mlp is None else FeedForwardConfig.from_dict(mlp, where)))
        bigram = _section(_section(d, "embedding", ""), "bigram", "embedding.")
        known = {"architecture", "architectures", "model_type", "vocab", "width", "norm", "canon", "layers", "embedding", "logit_softcap",
                 "max_position_embeddings", "eos_token_id"}
        return cls(
            vocab=require(d, "vocab", int), width=require(d, "width", int), norm_eps=require(_section(d, "norm", ""), "eps", float),
            canon_taps=require(_section(d, "canon", ""), "taps", int), bigram_buckets=require(bigram, "buckets", int),
            bigram_mul_prev=require(bigram, "mul_prev", int), bigram_mul_cur=require(bigram, "mul_cur", int),
            logit_softcap=require(d, "logit_softcap", float), layers=tuple(layers),
            max_position_embeddings=int(d.get("max_position_embeddings") or DEFAULT_MAX_POSITIONS),
            eos_token_id=int(d["eos_token_id"]) if isinstance(d.get("eos_token_id"), int) else -1,
            extra={k: v for k, v in d.items() if k not in known})

    @classmethod
    def from_json(cls, path: str | Path) -> "VasosunConfig":
        return cls.from_dict(read_config_json(path))

    def to_dict(self) -> dict[str, Any]:
        layers = [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict()} for l in self.layers]
        d: dict[str, Any] = {
            "architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
            "canon": {"taps": self.canon_taps},
            "embedding": {"bigram": {"buckets": self.bigram_buckets, "mul_prev": self.bigram_mul_prev, "mul_cur": self.bigram_mul_cur}},
            "logit_softcap": self.logit_softcap, "layers": layers}
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            d["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_id >= 0:
            d["eos_token_id"] = self.eos_token_id
        return d

    def save(self, folder: str | Path) -> None:
        write_config_json(folder, self.to_dict())


@register_architecture(ARCHITECTURE, model_types=("vasosun",), config_from_dict=VasosunConfig.from_dict)
def build_vasosun_spec(config: VasosunConfig) -> ModelSpec:
    W, eps = config.width, config.norm_eps

    def norm(name: str) -> PartSpec:  # one learned number for all channels
        return PartSpec("rmsnorm", {"dim": W, "eps": eps, "weight": name, "scalar": True})

    blocks: list[PartSpec] = []
    runs: list[RunSpec] = []
    ignorable: list[str] = []
    read_by_others = {l.mixer.kv_from for l in config.layers if isinstance(l.mixer, LatentAttentionConfig) and l.mixer.kv_from is not None}
    for i, layer in enumerate(config.layers):
        p = f"l{i}."
        params: dict[str, Any] = {
            "mixer": layer.mixer.part(W, eps, p + "mix."), "mixer_norm": norm(p + "norm1"), "mixer_out_norm": norm(p + "norm1b"),
            "hidden_size": W, "mixer_conv": p + "canon1", "conv_taps": config.canon_taps}
        if layer.mlp is not None:
            params.update(feed_forward=layer.mlp.part(W, p + "mlp."), ffn_norm=norm(p + "norm2"), ffn_out_norm=norm(p + "norm2b"),
                          ffn_conv=p + "canon2")
        else:
            ignorable += [p + "norm2", p + "norm2b", p + "canon2"]  # a layer without a feed-forward has no use for them
        blocks.append(PartSpec("sandwich_norm", params))
        # a layer that reads another layer's cached rows is a run that shares that layer's cache without writing it
        source = layer.mixer.kv_from if isinstance(layer.mixer, LatentAttentionConfig) else None
        if source is not None:
            runs.append(RunSpec(layer=i, cache=source, writes_cache=False))
        else:
            runs.append(RunSpec(layer=i, cache=i if i in read_by_others else None))
    return ModelSpec(
        vocab_size=config.vocab, hidden_size=W, embedding="embed", layers=blocks, final_norm=norm("final.norm"), lm_head="head",
        run_order=runs, max_positions=config.max_position_embeddings, eos_token_id=config.eos_token_id, ignorable_tensors=tuple(ignorable),
        embedding_transform=PartSpec("pair_hash_embedding", {
            "table": "bigram", "buckets": config.bigram_buckets, "mul_prev": config.bigram_mul_prev, "mul_cur": config.bigram_mul_cur,
            "hidden_size": W, "vocab_size": config.vocab}),
        logits_transform=PartSpec("softcap", {"cap": config.logit_softcap}))


# Named models of this design, so that the command lines can run them with random weights.
for _path in sorted(PRESET_DIR.glob("vasosun-*.json")):
    register_preset("vasosun", _path.stem, _path)
