"""Plain, slow Vasosun: whole sequences, no cache, one function per mechanism.

Vasosun is a decoder-only model whose layers put every sublayer between two norms of a single
learned number each, and whose sublayers read their normed input through a short causal
convolution over time that is added to it (y = h + conv(h), per channel):

    x <- x + N1b(mixer(C1(N1(x))));   x <- x + N2b(ff(C2(N2(x))))      (the second half where a layer has one)

A layer's mixer is one of three.  A sliding-window softmax attention without rotation, whose
queries grow with the logarithm of the position in steps and whose scores lose a logarithmic
distance term per head.  A latent attention (queries through a normed latent, keys and values
rebuilt from a normed latent plus one rotated key part for all heads; neighbouring entries turn
together, frequencies stretched between two wavelengths), which may read another layer's latents.
A gated delta rule (short convolutions and silu on q, k, v, unit q and k, one decay and one write
strength per head, the state corrected by what it already holds for the key).  The feed-forward
is a dense gated one or a set of routed experts chosen by softmax scores plus a correction, some of
which just hand their input on.  The embedding adds a row of a table hashed from the token pair;
the logits are bent through a tanh cap.

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


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.logaddexp(z, torch.zeros_like(z))


def scalar_norm(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    """The model's norm: unit root mean square, times one number for all channels."""
    return unit_rms(x, eps) * g.to(x.dtype).reshape(())


def causal_conv(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """h [T, C], w [C, taps]: out_t = sum_j w[:, j] h_(t - taps + 1 + j); rows before the start are zeros
    (the last column weighs the current token)."""
    T, taps = h.shape[0], w.shape[1]
    out = torch.zeros_like(h)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            out[back:] += w[:, j].to(h.dtype)[None, :] * h[: T - back]
    return out


def input_conv(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """What a sublayer reads: its normed input plus the convolution of it."""
    return h + causal_conv(h, w)


# ---------------------------------------------------------------------------
# embedding and output


def pair_rows(tokens: Sequence[int], buckets: int, mul_prev: int, mul_cur: int) -> list[int]:
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(buckets if t == 0 else (int(tokens[t - 1]) * mul_prev + int(tok) * mul_cur) % buckets)
    return rows


def embed(tokens: Sequence[int], weights: Weights, config: dict, dtype=torch.float64) -> torch.Tensor:
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    x = weights["embed"].to(dtype)[ids]
    b = config["embedding"]["bigram"]
    rows = torch.as_tensor(pair_rows(tokens, int(b["buckets"]), int(b["mul_prev"]), int(b["mul_cur"])), dtype=torch.long)
    return x + weights["bigram"].to(dtype)[rows]


def output_logits(x: torch.Tensor, weights: Weights, config: dict) -> torch.Tensor:
    y = scalar_norm(x, weights["final.norm"], float(config["norm"]["eps"])) @ weights["head"].to(x.dtype).T
    cap = float(config["logit_softcap"])
    return cap * torch.tanh(y / cap)


# ---------------------------------------------------------------------------
# windowed attention with a query temperature and a distance term


def query_temperature(positions: Sequence[int], coef: float, every: int) -> torch.Tensor:
    p = torch.as_tensor(list(positions), dtype=torch.float64)
    return 1.0 + coef * torch.log(torch.floor((p + 1.0) / every) + 1.0)


def softmax_over_visible(scores: torch.Tensor, visible: torch.Tensor) -> torch.Tensor:
    return torch.softmax(scores.masked_fill(~visible, float("-inf")), dim=-1)


def window_attention(h: torch.Tensor, positions: Sequence[int], m: dict, w: Weights, p: str) -> torch.Tensor:
    dt = h.dtype
    T, H, G, d, e = h.shape[0], int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ w[p + "q"].to(dt).T).view(T, H, d)
    k = (h @ w[p + "k"].to(dt).T).view(T, G, d)
    v = (h @ w[p + "v"].to(dt).T).view(T, G, e)
    if m.get("q_temp") is not None:
        q = q * query_temperature(positions, float(m["q_temp"]["coef"]), int(m["q_temp"]["every"])).to(dt)[:, None, None]
    pos = torch.as_tensor(list(positions), dtype=torch.long)
    dist = pos[:, None] - pos[None, :]
    visible = dist >= 0
    if m.get("mask") is not None:  # a configuration without one: every earlier key
        visible = visible & (dist < int(m["mask"]["size"]))
    far = dist.clamp(min=0).to(dt)
    r1, r2 = w[p + "r1"].to(dt), w[p + "r2"].to(dt)
    heads = []
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * float(m["scale"]) - r1[a] * torch.log1p(r2[a] * far)
        heads.append(softmax_over_visible(s, visible) @ v[:, g])
    return torch.cat(heads, dim=-1) @ w[p + "o"].to(dt).T


# ---------------------------------------------------------------------------
# latent attention


def stretched_frequencies(base: float, dims: int, s: Optional[dict]) -> tuple[torch.Tensor, float]:
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.as_tensor(float(base), dtype=torch.float64) ** (-2.0 * i / dims)
    if s is None:
        return f, 1.0
    factor, original = float(s["factor"]), float(s["original"])

    def index_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(float(s["fast"]))), 0)
    hi = min(math.ceil(index_of(float(s["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_neighbours(x: torch.Tensor, positions: Sequence[int], freq: torch.Tensor, magnitude: float) -> torch.Tensor:
    """x [T, ..., n]: entries 2i and 2i+1 (i < len(freq)) turn together by position * freq[i]; cosine and
    sine carry `magnitude`; the entries behind stay."""
    n = 2 * freq.numel()
    if n == 0:
        return x
    ang = torch.as_tensor(list(positions), dtype=torch.float64)[:, None] * freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [freq.numel()]
    c = (torch.cos(ang) * magnitude).to(x.dtype).view(shape)
    s = (torch.sin(ang) * magnitude).to(x.dtype).view(shape)
    u, v = x[..., 0:n:2], x[..., 1:n:2]
    turned = torch.stack([u * c - v * s, v * c + u * s], dim=-1).flatten(-2)
    return torch.cat([turned, x[..., n:]], dim=-1)


def latent_rows(h: torch.Tensor, positions: Sequence[int], m: dict, w: Weights, p: str, eps: float) -> tuple[torch.Tensor, torch.Tensor]:
    """What a latent attention layer caches per token: the normed latent and the rotated key part."""
    dt = h.dtype
    R = int(m["kv_rank"])
    rows = h @ w[p + "dkv"].to(dt).T
    c = unit_rms(rows[:, :R], eps) * w[p + "dkv.norm"].to(dt)
    freq, mag = stretched_frequencies(float(m["rot"]["base"]), int(m["rot"]["dims"]), m["rot"].get("scaling"))
    return c, rotate_neighbours(rows[:, R:], positions, freq, mag)


def latent_attention(h: torch.Tensor, positions: Sequence[int], m: dict, w: Weights, p: str, eps: float,
                     c: torch.Tensor, k_rot: torch.Tensor) -> torch.Tensor:
    dt = h.dtype
    T, H, d, r, e, R = h.shape[0], int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    cq = unit_rms(h @ w[p + "dq"].to(dt).T, eps) * w[p + "dq.norm"].to(dt)
    q = (cq @ w[p + "uq"].to(dt).T).view(T, H, d + r)
    freq, mag = stretched_frequencies(float(m["rot"]["base"]), int(m["rot"]["dims"]), m["rot"].get("scaling"))
    q_plain, q_rot = q[..., :d], rotate_neighbours(q[..., d:], positions, freq, mag)
    k_plain = (c @ w[p + "uk"].to(dt).T).view(T, H, d)
    v = (c @ w[p + "uv"].to(dt).T).view(T, H, e)
    visible = torch.ones(T, T, dtype=torch.bool).tril()
    heads = []
    for a in range(H):
        s = (q_plain[:, a] @ k_plain[:, a].T + q_rot[:, a] @ k_rot.T) * float(m["scale"])
        heads.append(softmax_over_visible(s, visible) @ v[:, a])
    return torch.cat(heads, dim=-1) @ w[p + "o"].to(dt).T


# ---------------------------------------------------------------------------
# gated delta rule


def unit_length(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt(x.pow(2).sum(-1, keepdim=True) + 1e-6)


def delta_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, beta: torch.Tensor) -> torch.Tensor:
    """One head.  q, k [T, d], v [T, e], decay and beta [T].  S starts at zero; per token:
    S <- decay S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T, d, e = q.shape[0], q.shape[1], v.shape[1]
    S = torch.zeros(d, e, dtype=q.dtype)
    out = torch.zeros(T, e, dtype=q.dtype)
    for t in range(T):
        S = decay[t] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def delta_mixer(h: torch.Tensor, m: dict, w: Weights, p: str, eps: float) -> torch.Tensor:
    dt = h.dtype
    T, H, G, d, e = h.shape[0], int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])

    def short(name: str) -> torch.Tensor:
        return silu(causal_conv(h @ w[p + name].to(dt).T, w[p + name + ".conv"]))

    q = unit_length(short("q").view(T, G, d)) * d ** -0.5
    k = unit_length(short("k").view(T, G, d))
    v = short("v").view(T, H, e)
    beta = torch.sigmoid(h @ w[p + "b"].to(dt).T)
    decay = torch.exp(-torch.exp(w[p + "A_log"].to(dt)) * softplus(h @ w[p + "a"].to(dt).T + w[p + "dt_bias"].to(dt)))
    gate = silu(h @ w[p + "g"].to(dt).T).view(T, H, e)
    heads = []
    for a in range(H):
        g = a // (H // G)
        o = delta_recurrence(q[:, g], k[:, g], v[:, a], decay[:, a], beta[:, a])
        heads.append(unit_rms(o, eps) * w[p + "norm"].to(dt) * gate[:, a])
    return torch.cat(heads, dim=-1) @ w[p + "o"].to(dt).T


# ---------------------------------------------------------------------------
# feed-forwards


def dense_ff(h: torch.Tensor, w: Weights, p: str) -> torch.Tensor:
    dt = h.dtype
    return (silu(h @ w[p + "gate"].to(dt).T) * (h @ w[p + "up"].to(dt).T)) @ w[p + "down"].to(dt).T


def route(h: torch.Tensor, mlp: dict, w: Weights, p: str) -> tuple[torch.Tensor, torch.Tensor]:
    """Chosen experts [T, top] (an index >= experts is an identity expert) and their weights."""
    dt = h.dtype
    s = torch.softmax(h @ w[p + "router"].to(dt).T, dim=-1)
    choice = s + w[p + "correction"].to(dt)
    chosen = torch.topk(choice, int(mlp["router"]["top"]), dim=-1).indices
    return chosen, torch.gather(s, 1, chosen)


def routed_ff(h: torch.Tensor, mlp: dict, w: Weights, p: str, chosen: Optional[torch.Tensor] = None,
              weights: Optional[torch.Tensor] = None) -> torch.Tensor:
    dt = h.dtype
    E = int(mlp["router"]["experts"])
    if chosen is None:
        chosen, weights = route(h, mlp, w, p)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t].tolist(), weights[t]):
            if e >= E:
                out[t] += a * h[t]
            else:
                out[t] += a * (gelu_erf(h[t] @ w[f"{p}e{e}.up"].to(dt).T) @ w[f"{p}e{e}.down"].to(dt).T)
    return out


# ---------------------------------------------------------------------------
# the model


def forward_stream(tokens: Sequence[int], weights: Weights, config: dict, dtype=torch.float64,
                   rounding: Optional[Callable[[torch.Tensor], torch.Tensor]] = None) -> list[torch.Tensor]:
    """The residual stream [T, width] after the embedding and after every layer.  `rounding`, if
    given, is applied to what every sublayer reads (to see what a narrower number format does)."""
    eps = float(config["norm"]["eps"])
    rd = rounding if rounding is not None else (lambda t: t)
    positions = list(range(len(tokens)))
    x = embed(tokens, weights, config, dtype)
    streams = [x]
    latents: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}
    for i, layer in enumerate(config["layers"]):
        p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        h = rd(input_conv(scalar_norm(x, weights[p + "norm1"], eps), weights[p + "canon1"]))
        if kind == "attention":
            y = window_attention(h, positions, m, weights, p + "mix.")
        elif kind == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                latents[i] = latent_rows(h, positions, m, weights, p + "mix.", eps)
                src = i
            y = latent_attention(h, positions, m, weights, p + "mix.", eps, *latents[int(src)])
        elif kind == "delta":
            y = delta_mixer(h, m, weights, p + "mix.", eps)
        else:
            raise ValueError(f"unknown mixer {kind!r}")
        x = x + scalar_norm(y, weights[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rd(input_conv(scalar_norm(x, weights[p + "norm2"], eps), weights[p + "canon2"]))
            f = dense_ff(h, weights, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(h, mlp, weights, p + "mlp.")
            x = x + scalar_norm(f, weights[p + "norm2b"], eps)
        streams.append(x)
    return streams


def forward_logits(tokens: Sequence[int], weights: Weights, config: dict, dtype=torch.float64,
                   rounding: Optional[Callable[[torch.Tensor], torch.Tensor]] = None) -> torch.Tensor:
    return output_logits(forward_stream(tokens, weights, config, dtype, rounding)[-1], weights, config)
