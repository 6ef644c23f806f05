"""Rotary position encoding (rotate-half pairing) as a part of its own."""

from __future__ import annotations

import math
from typing import Any, Mapping, Optional

import torch

from tokensprint_b200 import ops
from tokensprint_b200.parts.base import BuildContext, PositionEncoding, StepContext, register_part


def rope_inverse_frequencies(dim: int, theta: float) -> torch.Tensor:
    """inv_freq[j] = 1 / theta^(2j/dim), j = 0..dim/2-1, float32 on the host.

    The reference's formula and dtype (engine/nn/rope.py:28-29).
    """
    idx = torch.arange(0, dim, step=2, dtype=torch.float32)
    return 1.0 / (theta ** (idx / dim))


def rope_inverse_frequencies_exact(dim: int, theta: float) -> torch.Tensor:
    """theta^(-2j/dim), j = 0..dim/2-1, worked out in float64 and rounded once to float32."""
    idx = torch.arange(0, dim, step=2, dtype=torch.float64)
    return torch.pow(torch.tensor(float(theta), dtype=torch.float64), -idx / dim).to(torch.float32)


def scaled_frequencies(dim: int, theta: float, scaling: Optional[Mapping[str, Any]]) -> tuple[torch.Tensor, float]:
    """Inverse frequencies theta^(-2j/dim) stretched for contexts longer than the one a model was
    trained on, in float64, and the magnitude that cosines and sines are multiplied by.

    `scaling` None: the plain frequencies, magnitude 1.  Otherwise a mapping with `kind`:

    "yarn" (factor, original, fast, slow): the pair index at which a wave makes t turns over
    `original` positions is i(t) = dim ln(original / (2 pi t)) / (2 ln theta); with lo = max(floor(i(fast)), 0),
    hi = min(ceil(i(slow)), dim - 1) and ramp_j = clamp((j - lo) / max(hi - lo, 0.001), 0, 1) the
    frequency becomes f_j / factor * ramp_j + f_j (1 - ramp_j); the magnitude is 0.1 ln(factor) + 1.

    "llama3" (factor, low, high, original): with wavelength l = 2 pi / f, f stays where
    l < original / high, becomes f / factor where l > original / low, and between the two, with
    s = (original / l - low) / (high - low), (1 - s) f / factor + s f; magnitude 1."""
    j = torch.arange(dim // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * j / dim)
    if scaling is None:
        return f, 1.0
    kind = scaling.get("kind")
    factor, original = float(scaling["factor"]), float(scaling["original"])
    if kind == "yarn":
        def index_of(turns: float) -> float:
            return dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

        lo = max(math.floor(index_of(float(scaling["fast"]))), 0)
        hi = min(math.ceil(index_of(float(scaling["slow"]))), dim - 1)
        ramp = torch.clamp((j - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0
    if kind == "llama3":
        low, high = float(scaling["low"]), float(scaling["high"])
        wavelength = 2.0 * math.pi / f
        s = (original / wavelength - low) / (high - low)
        between = (1.0 - s) * f / factor + s * f
        return torch.where(wavelength < original / high, f, torch.where(wavelength > original / low, f / factor, between)), 1.0
    raise ValueError(f"rotary scaling kind must be 'yarn' or 'llama3', got {kind!r}")


@register_part("position_encoding", "rotary")
class RotaryEncoding(PositionEncoding):
    """x'[j] = x[j] cos - x[j+r/2] sin, x'[j+r/2] = x[j+r/2] cos + x[j] sin over the first
    `dim` (= r) entries of each head, angle = position * inv_freq[j] in float32
    (engine/nn/rope.py:105-123, engine/kernels/triton/rope.py:22-65).  The rotation
    itself runs inside the fused q/k kernel; this part owns the frequencies.

    `pairing` "half" (the default) is the above; "neighbours" turns entry 2i with entry 2i+1 by
    the same angles (mixers whose kernels take a pairing ask for it through `pairing`; the fused
    q/k kernels of the attention mixer know the half pairing only, so `rotary_inv_freq()` answers
    None for the other and that mixer falls back to `apply`, which this part does not offer).
    `exact_frequencies`: the inverse frequencies are worked out in float64 before they are rounded.
    `scaling`: stretched frequencies and a magnitude on cosines and sines (scaled_frequencies); the
    fused kernels, which make their own cosines and sines, are then offered the frequencies only
    while the magnitude is 1, and `rotary_table` serves every case."""

    graph_safe = True

    def __init__(self, ctx: BuildContext, *, dim: int, theta: float, pairing: str = "half", exact_frequencies: bool = False,
                 scaling: Optional[Mapping[str, Any]] = None) -> None:
        if dim % 2:
            raise ValueError(f"rotary width must be even, got {dim}")
        if pairing not in ops.ROTARY_PAIRINGS:
            raise ValueError(f"rotary pairing must be one of {sorted(ops.ROTARY_PAIRINGS)}, got {pairing!r}")
        self.dim, self.theta, self.pairing = int(dim), float(theta), pairing
        self.scaling = None if scaling is None else dict(scaling)
        exact, self.magnitude = scaled_frequencies(self.dim, self.theta, self.scaling)
        if self.scaling is not None:
            self.inv_freq = exact.to(torch.float32).to(ctx.device)
        else:
            make = rope_inverse_frequencies_exact if exact_frequencies else rope_inverse_frequencies
            self.inv_freq = make(self.dim, self.theta).to(ctx.device)
        self.inv_freq64 = exact.to(ctx.device)
        self._key = ("rotary_table", self.dim, self.theta, None if self.scaling is None else tuple(sorted(self.scaling.items())))

    def rotary_inv_freq(self) -> Optional[torch.Tensor]:
        return self.inv_freq if self.pairing == "half" and self.magnitude == 1.0 else None

    def rotary_table(self, step: StepContext) -> torch.Tensor:
        """[T, dim/2, 2] float32: magnitude * (cos, sin) of the step's angles, which are formed in
        float64 from the float64 frequencies; made by the first layer of a step that asks and used
        by all layers with the same width, base and scaling."""
        table = step.shared.get(self._key)
        if table is None:
            table = step.shared[self._key] = ops.rope_table(step.positions, self.inv_freq64, self.magnitude, step.num_tokens)
        return table

    def frequencies(self) -> torch.Tensor:
        """[dim/2] float32 inverse frequencies, whatever the pairing (for kernels that take one)."""
        return self.inv_freq

    def rotary_cos_sin(self, step: StepContext) -> Optional[torch.Tensor]:
        """The table of the step, made by the first layer that asks and used by all layers with the
        same width and base (angles, cosines and sines in float32, as in the rotating kernels)."""
        key = ("rotary_cos_sin", self.dim, self.theta)
        table = step.shared.get(key)
        if table is None:
            table = step.shared[key] = ops.rope_cos_sin(step.positions, self.inv_freq, step.num_tokens)
        return table
