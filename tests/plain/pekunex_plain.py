"""Plain, slow Pekunex: whole sequences, no cache, one function per mechanism.

Pekunex is a decoder-only model of pre-normed layers (x <- x + mixer(norm1(x)), then
x <- x + ff(norm2(x)) where the layer has a feed-forward).  A layer's mixer is one of three:
a softmax attention with biased projections, a rotation whose frequencies are stretched smoothly
between two wavelengths and whose cosines and sines carry a magnitude, q and k divided by their
root mean square after the rotation, scores bent through a tanh cap and an output gate; a pair of
mixers side by side whose outputs are added with fixed weights (a softmax attention with a learned
sink per head and piecewise stretched frequencies beside a matrix memory with exponential gates
kept in range by a running maximum); or a selective state-space recurrence (scalar decay per head,
short causal convolution on its inputs, gated and normed in groups on the way out).  A layer may
borrow another layer's weights.  The embedding rows and the logits are multiplied by constants.

Everything here runs on whole sequences in one dtype (float64 by default) on the CPU and shares
no code with the engine under test.  `config` is the content of a config.json as a dict,
`weights` a dict of tensors under the checkpoint's names.
"""

from __future__ import annotations

import math
from typing import Callable, Mapping, Optional, Sequence

import torch

Weights = Mapping[str, torch.Tensor]


# ---------------------------------------------------------------------------
# small functions


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """Rows divided by their root mean square, eps under the root."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * w


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.logaddexp(z, torch.zeros_like(z))


def embed(tokens: Sequence[int], weights: Weights, config: dict, dtype=torch.float64) -> torch.Tensor:
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    return weights["embed"].to(dtype)[ids] * float(config["embedding"]["scale"])


def weight_owner(config: dict, i: int) -> int:
    """The layer whose tensors layer i uses (itself unless it names another)."""
    j = config["layers"][i].get("weights_of")
    return i if j is None else int(j)


# ---------------------------------------------------------------------------
# rotation frequencies


def base_frequencies(base: float, dims: int) -> torch.Tensor:
    i = torch.arange(dims // 2, dtype=torch.float64)
    return torch.as_tensor(float(base), dtype=torch.float64) ** (-2.0 * i / dims)


def smooth_stretch(base: float, dims: int, s: dict) -> tuple[torch.Tensor, float]:
    """Frequencies divided by `factor` where the pair index lies beyond the index that `slow` turns
    of the original length correspond to, untouched before the index of `fast` turns, a straight
    ramp between; and the magnitude that multiplies cosines and sines."""
    f = base_frequencies(base, dims)
    factor, original = float(s["factor"]), float(s["original"])

    def index_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(float(s["fast"]))), 0)
    hi = min(math.ceil(index_of(float(s["slow"]))), dims - 1)
    i = torch.arange(dims // 2, dtype=torch.float64)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def piecewise_stretch(base: float, dims: int, s: dict) -> tuple[torch.Tensor, float]:
    """Frequencies kept where the wavelength is shorter than original/high, divided by `factor`
    where it is longer than original/low, blended in between."""
    f = base_frequencies(base, dims)
    factor, low, high, original = float(s["factor"]), float(s["low"]), float(s["high"]), float(s["original"])
    wavelength = 2.0 * math.pi / f
    blend = (original / wavelength - low) / (high - low)
    mid = (1.0 - blend) * f / factor + blend * f
    out = torch.where(wavelength < original / high, f, torch.where(wavelength > original / low, f / factor, mid))
    return out, 1.0


def rotate_halves(x: torch.Tensor, positions: Sequence[int], freq: torch.Tensor, magnitude: float) -> torch.Tensor:
    """x [T, heads, n]: entry i < len(freq) is paired with entry i + len(freq); the pair turns by
    position * freq[i], and cosine and sine carry `magnitude`; the rest of a head stays."""
    half = freq.numel()
    if half == 0:
        return x
    ang = torch.as_tensor(list(positions), dtype=torch.float64)[:, None] * freq[None, :]
    c = (torch.cos(ang) * magnitude).to(x.dtype)[:, None, :]
    s = (torch.sin(ang) * magnitude).to(x.dtype)[:, None, :]
    u, v = x[..., :half], x[..., half:2 * half]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., 2 * half:]], dim=-1)


# ---------------------------------------------------------------------------
# softmax attention, in the two forms of the design


def causal_weights(scores: torch.Tensor, sink: Optional[float] = None) -> torch.Tensor:
    """scores [T, T] (query, key): softmax over the keys j <= i; with `sink` the denominator also
    holds exp(sink)."""
    T = scores.shape[0]
    visible = torch.ones(T, T, dtype=torch.bool).tril()
    top = scores.masked_fill(~visible, -math.inf).max(-1, keepdim=True).values
    if sink is not None:
        top = torch.clamp(top, min=sink)
    e = torch.where(visible, torch.exp(scores - top), torch.zeros_like(scores))
    denom = e.sum(-1, keepdim=True)
    if sink is not None:
        denom = denom + torch.exp(sink - top)
    return e / denom


def capped_attention(h: torch.Tensor, positions: Sequence[int], m: dict, prefix: str, weights: Weights, eps: float) -> torch.Tensor:
    """Biased projections, smooth-stretched rotation with a magnitude, unit-rms q and k after the
    rotation, tanh-capped scores, sigmoid output gate."""
    T, dt = h.shape[0], h.dtype
    H, G, d, e = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    w = lambda name: weights[prefix + name].to(dt)
    q = (h @ w("q").T + w("q.b")).reshape(T, H, d)
    k = (h @ w("k").T + w("k.b")).reshape(T, G, d)
    v = (h @ w("v").T + w("v.b")).reshape(T, G, e)
    rot = m.get("rot")
    if rot is not None and int(rot["dims"]) > 0:
        if rot.get("scaling") is not None:
            freq, magnitude = smooth_stretch(float(rot["base"]), int(rot["dims"]), rot["scaling"])
        else:
            freq, magnitude = base_frequencies(float(rot["base"]), int(rot["dims"])), 1.0
        q, k = rotate_halves(q, positions, freq, magnitude), rotate_halves(k, positions, freq, magnitude)
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    cap = float(m["softcap"]) if m.get("softcap") else None
    out = torch.empty(T, H, e, dtype=dt)
    for head in range(H):
        g = head // (H // G)
        scores = (q[:, head] @ k[:, g].T) * float(m["scale"])
        if cap is not None:
            scores = cap * torch.tanh(scores / cap)
        out[:, head] = causal_weights(scores) @ v[:, g]
    gate = torch.sigmoid(h @ w("g").T)
    return (out.reshape(T, H * e) * gate) @ w("o").T


def sink_attention(h: torch.Tensor, positions: Sequence[int], m: dict, prefix: str, weights: Weights) -> torch.Tensor:
    """No biases, piecewise-stretched rotation, a learned sink per head in the denominator."""
    T, dt = h.shape[0], h.dtype
    H, G, d, e = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    w = lambda name: weights[prefix + name].to(dt)
    q = (h @ w("q").T).reshape(T, H, d)
    k = (h @ w("k").T).reshape(T, G, d)
    v = (h @ w("v").T).reshape(T, G, e)
    rot = m.get("rot")
    if rot is not None and int(rot["dims"]) > 0:
        if rot.get("scaling") is not None:
            freq, magnitude = piecewise_stretch(float(rot["base"]), int(rot["dims"]), rot["scaling"])
        else:
            freq, magnitude = base_frequencies(float(rot["base"]), int(rot["dims"])), 1.0
        q, k = rotate_halves(q, positions, freq, magnitude), rotate_halves(k, positions, freq, magnitude)
    sinks = w("sink")
    out = torch.empty(T, H, e, dtype=dt)
    for head in range(H):
        g = head // (H // G)
        scores = (q[:, head] @ k[:, g].T) * float(m["scale"])
        out[:, head] = causal_weights(scores, sink=float(sinks[head])) @ v[:, g]
    return out.reshape(T, H * e) @ w("o").T


# ---------------------------------------------------------------------------
# matrix memory with exponential gates


def matrix_memory_gates(h: torch.Tensor, m: dict, prefix: str, weights: Weights) -> tuple[torch.Tensor, torch.Tensor]:
    """[T, heads] logarithms of the input gate and of the forget gate, both bent through a tanh cap."""
    dt, cap = h.dtype, float(m["gate_cap"])
    w = lambda name: weights[prefix + name].to(dt)
    log_i = cap * torch.tanh((h @ w("i").T + w("i.b")) / cap)
    log_f = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w("f").T + w("f.b")) / cap))
    return log_i, log_f


def matrix_memory_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, log_i: torch.Tensor, log_f: torch.Tensor,
                             state: Optional[tuple[torch.Tensor, torch.Tensor, float]] = None):
    """One head, token by token.  q, k [T, d] (q already scaled); v [T, e]; log_i, log_f [T].
    The memory S [d, e], the normaliser n [d] and the running maximum m (0 before the first token)."""
    T, d = q.shape
    e = v.shape[1]
    if state is None:
        S, n, m = torch.zeros(d, e, dtype=q.dtype), torch.zeros(d, dtype=q.dtype), 0.0
    else:
        S, n, m = state[0].clone(), state[1].clone(), float(state[2])
    out = torch.empty(T, e, dtype=q.dtype)
    for t in range(T):
        m_new = max(float(log_f[t]) + m, float(log_i[t]))
        keep, take = math.exp(float(log_f[t]) + m - m_new), math.exp(float(log_i[t]) - m_new)
        S = keep * S + take * k[t][:, None] * v[t][None, :]
        n = keep * n + take * k[t]
        m = m_new
        out[t] = (S.T @ q[t]) / (max(abs(float(n @ q[t])), math.exp(-m)) + 1e-6)
    return out, (S, n, m)


def matrix_memory(h: torch.Tensor, m: dict, prefix: str, weights: Weights, eps: float) -> torch.Tensor:
    T, dt = h.shape[0], h.dtype
    H, d, e = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    w = lambda name: weights[prefix + name].to(dt)
    q = (h @ w("q").T).reshape(T, H, d) * d ** -0.5
    k = (h @ w("k").T).reshape(T, H, d)
    v = (h @ w("v").T).reshape(T, H, e)
    log_i, log_f = matrix_memory_gates(h, m, prefix, weights)
    out = torch.empty(T, H, e, dtype=dt)
    for head in range(H):
        o, _ = matrix_memory_recurrence(q[:, head], k[:, head], v[:, head], log_i[:, head], log_f[:, head])
        out[:, head] = unit_rms(o, eps)
    y = out.reshape(T, H * e) * w("norm") * torch.sigmoid(h @ w("g").T)
    return y @ w("o").T


def side_by_side(h: torch.Tensor, positions: Sequence[int], m: dict, prefix: str, weights: Weights, eps: float) -> torch.Tensor:
    left = sink_attention(h, positions, m["left"], prefix + "left.", weights)
    right = matrix_memory(h, m["right"], prefix + "right.", weights, eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


# ---------------------------------------------------------------------------
# selective state-space recurrence


def short_convolution(x: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor, before: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, C]; taps [C, K], the last column weighs the current token; zeros (or `before`
    [K-1, C]) stand before the first token."""
    T, C = x.shape
    K = taps.shape[1]
    pad = torch.zeros(K - 1, C, dtype=x.dtype) if before is None else before.to(x.dtype)
    xp = torch.cat([pad, x], dim=0)
    out = bias[None, :].expand(T, C).clone()
    for j in range(K):
        out = out + xp[j:j + T] * taps[:, j][None, :]
    return out


def state_space_recurrence(x: torch.Tensor, B: torch.Tensor, C: torch.Tensor, dt: torch.Tensor, a: float, D: float,
                           state: Optional[torch.Tensor] = None) -> tuple[torch.Tensor, torch.Tensor]:
    """One head.  x [T, e]; B, C [T, N]; dt [T] (after softplus); a = exp(A_log) > 0.
    S [N, e]: S_t = exp(-a dt_t) S_(t-1) + dt_t B_t x_t^T;  y_t = S_t^T C_t + D x_t."""
    T, e = x.shape
    S = torch.zeros(B.shape[1], e, dtype=x.dtype) if state is None else state.clone()
    out = torch.empty(T, e, dtype=x.dtype)
    for t in range(T):
        S = math.exp(-a * float(dt[t])) * S + float(dt[t]) * B[t][:, None] * x[t][None, :]
        out[t] = S.T @ C[t] + D * x[t]
    return out, S


def state_space(h: torch.Tensor, m: dict, prefix: str, weights: Weights, eps: float) -> torch.Tensor:
    T, dtp = h.shape[0], h.dtype
    H, e, N, G = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    parts = int(m["norm_groups"])
    inner = H * e
    w = lambda name: weights[prefix + name].to(dtp)
    proj = h @ w("in").T
    z, xbc, dt_raw = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_convolution(xbc, w("conv"), w("conv.b")))
    x = xbc[:, :inner].reshape(T, H, e)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt_raw + w("dt_bias"))
    a, D = torch.exp(w("A_log")), w("D")
    y = torch.empty(T, H, e, dtype=dtp)
    for head in range(H):
        g = head // (H // G)
        y[:, head], _ = state_space_recurrence(x[:, head], B[:, g], C[:, g], dt[:, head], float(a[head]), float(D[head]))
    y = y.reshape(T, inner) * silu(z)
    y = unit_rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w("norm")
    return y @ w("o").T


# ---------------------------------------------------------------------------
# feed-forward, a layer and the model


def feed_forward(h: torch.Tensor, prefix: str, weights: Weights) -> torch.Tensor:
    dt = h.dtype
    w = lambda name: weights[prefix + name].to(dt)
    return (silu(h @ w("gate").T) * (h @ w("up").T)) @ w("down").T


def mixer(h: torch.Tensor, positions: Sequence[int], entry: dict, prefix: str, weights: Weights, eps: float) -> torch.Tensor:
    kind = entry["type"]
    if kind == "attention":
        return capped_attention(h, positions, entry["mixer"], prefix, weights, eps)
    if kind == "parallel":
        return side_by_side(h, positions, entry["mixer"], prefix, weights, eps)
    if kind == "mamba2":
        return state_space(h, entry["mixer"], prefix, weights, eps)
    raise ValueError(f"unknown mixer {kind!r}")


def layer(x: torch.Tensor, positions: Sequence[int], i: int, config: dict, weights: Weights) -> torch.Tensor:
    entry, eps, dt = config["layers"][i], float(config["norm"]["eps"]), x.dtype
    p = f"l{weight_owner(config, i)}."
    x = x + mixer(norm(x, weights[p + "norm1"].to(dt), eps), positions, entry, p + "mix.", weights, eps)
    if entry.get("mlp") is not None:
        x = x + feed_forward(norm(x, weights[p + "norm2"].to(dt), eps), p + "mlp.", weights)
    return x


def forward_stream(tokens: Sequence[int], weights: Weights, config: dict, dtype=torch.float64,
                   after_run: Optional[Callable[[int, torch.Tensor], None]] = None) -> torch.Tensor:
    positions = list(range(len(tokens)))
    x = embed(tokens, weights, config, dtype)
    for i in range(len(config["layers"])):
        x = layer(x, positions, i, config, weights)
        if after_run is not None:
            after_run(i, x)
    return x


def forward_logits(tokens: Sequence[int], weights: Weights, config: dict, dtype=torch.float64) -> torch.Tensor:
    x = forward_stream(tokens, weights, config, dtype)
    x = norm(x, weights["final.norm"].to(dtype), float(config["norm"]["eps"]))
    return (x @ weights["head"].to(dtype).T) * float(config.get("logit_scale", 1.0))
