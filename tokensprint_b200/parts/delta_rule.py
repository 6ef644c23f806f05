"""The gated delta rule as a mixer part: a recurrence whose state is corrected, token by token, by
what it already returns for the new key; state and the short convolutions' kept inputs per request
live in a float32 state slot of the cache."""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from tokensprint_b200 import ops
from tokensprint_b200.parts.base import BuildContext, CacheNeed, LayerCache, Mixer, StepContext, TensorSpec, register_part
from tokensprint_b200.parts.linear import linear, linear_float32_out


@register_part("mixer", "gated_delta_rule")
class GatedDeltaRule(Mixer):
    """With H heads of value width e, G <= H heads of q and k of width d (head h reads q/k head
    h // (H / G)), for the tokens of a sequence in order:

        q = silu(conv(W_q x)),  k = silu(conv(W_k x)),  v = silu(conv(W_v x))     short causal convolutions per
                                                                                channel, `taps` wide, no bias
        q <- q / sqrt(sum q^2 + unit_eps) * q_scale,   k <- k / sqrt(sum k^2 + unit_eps)     per head
        beta = sigmoid(W_b x),   g = exp(-exp(A_log_h) * softplus(W_a x + dt_bias_h))         per head
        S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q                      S [d, e], zero at first
        y = W_o ( concat over heads of  o * rsqrt(mean(o^2) + norm_eps) * w_norm * silu(W_g x) )

    Parameters: `hidden_size`, `num_heads`, `num_qk_heads`, `key_dim`, `value_dim`, `taps`, `norm_eps`,
    `unit_eps` (default 1e-6), `q_scale` (default key_dim^-0.5) and the tensors' names.  One product
    gives [q | k | v | output gate] in the compute dtype, a second one the raw write-strength and
    decay rows, whose sums leave in float32.  The convolutions with their silu, unit lengths, beta,
    the decay, the state, the recurrence and the head norm are float32 whatever the compute dtype.
    The state slot holds the state [H, e, d] (value column by value column) followed by the last
    taps - 1 inputs of the convolutions [taps - 1, 2 G d + H e], oldest first; zeros before the first
    token, so prompts may be cut anywhere."""

    graph_safe = True
    reads_through_ops = True

    def __init__(self, ctx: BuildContext, *, hidden_size: int, num_heads: int, num_qk_heads: int, key_dim: int, value_dim: int, taps: int,
                 norm_eps: float, q: str, k: str, v: str, q_conv: str, k_conv: str, v_conv: str, beta: str, decay: str, a_log: str,
                 dt_bias: str, gate: str, norm: str, o: str, unit_eps: float = 1e-6, q_scale: Optional[float] = None) -> None:
        self.hidden_size, self.num_heads, self.num_qk_heads = int(hidden_size), int(num_heads), int(num_qk_heads)
        self.key_dim, self.value_dim, self.taps = int(key_dim), int(value_dim), int(taps)
        self.norm_eps, self.unit_eps = float(norm_eps), float(unit_eps)
        if min(self.num_heads, self.num_qk_heads, self.key_dim, self.value_dim, self.taps) < 1 or self.num_heads % self.num_qk_heads:
            raise ValueError("gated delta rule: sizes must be positive and heads a multiple of the q/k heads")
        if self.key_dim > ops.DELTA_MAX_KEY_DIM:
            raise ValueError(f"gated delta rule: key_dim {key_dim} exceeds the kernel's {ops.DELTA_MAX_KEY_DIM}")
        self.q_scale = float(q_scale) if q_scale is not None else float(self.key_dim) ** -0.5
        self.qk_width, self.v_width = self.num_qk_heads * self.key_dim, self.num_heads * self.value_dim
        self.channels = 2 * self.qk_width + self.v_width
        self.memory_floats = self.num_heads * self.key_dim * self.value_dim
        self.names = {"q": q, "k": k, "v": v, "q_conv": q_conv, "k_conv": k_conv, "v_conv": v_conv, "beta": beta, "decay": decay,
                      "a_log": a_log, "dt_bias": dt_bias, "gate": gate, "norm": norm, "o": o}
        self.in_weight: Optional[torch.Tensor] = None    # [q | k | v | gate] stacked
        self.gate_rows: Optional[torch.Tensor] = None    # [beta | decay] stacked
        self.o_weight: Optional[torch.Tensor] = None

    def first_weight(self) -> Optional[torch.Tensor]:
        return self.in_weight

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="none", state_shape=(self.memory_floats + (self.taps - 1) * self.channels,), state_dtype=torch.float32)

    def tensor_specs(self) -> list[TensorSpec]:
        W, n, H = self.hidden_size, self.names, self.num_heads
        return [TensorSpec(n["q"], (self.qk_width, W)), TensorSpec(n["k"], (self.qk_width, W)), TensorSpec(n["v"], (self.v_width, W)),
                TensorSpec(n["q_conv"], (self.qk_width, self.taps), "vector"), TensorSpec(n["k_conv"], (self.qk_width, self.taps), "vector"),
                TensorSpec(n["v_conv"], (self.v_width, self.taps), "vector"), TensorSpec(n["beta"], (H, W)), TensorSpec(n["decay"], (H, W)),
                TensorSpec(n["a_log"], (H,), "vector"), TensorSpec(n["dt_bias"], (H,), "vector"), TensorSpec(n["gate"], (self.v_width, W)),
                TensorSpec(n["norm"], (self.value_dim,), "vector"), TensorSpec(n["o"], (W, self.v_width))]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        self.in_weight = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]], tensors[n["gate"]]], dim=0).contiguous()
        self.gate_rows = torch.cat([tensors[n["beta"]], tensors[n["decay"]]], dim=0).contiguous()
        # the three convolutions as one, tap by tap [taps, channels], as the kernel reads them
        self.conv_weight = torch.cat([tensors[n["q_conv"]], tensors[n["k_conv"]], tensors[n["v_conv"]]], dim=0).t().contiguous()
        self.a_log, self.dt_bias = tensors[n["a_log"]], tensors[n["dt_bias"]]
        self.norm_weight, self.o_weight = tensors[n["norm"]], tensors[n["o"]]

    def forward(self, x: torch.Tensor, step: StepContext, cache: LayerCache) -> torch.Tensor:
        if cache.state is None:
            raise ops.KernelError("gated delta rule: this mixer needs a state slot per request (none was bound to its run)")
        if not cache.writes:
            raise ops.KernelError("gated delta rule: a run cannot read another run's state")
        T, H, G, d, e = x.shape[0], self.num_heads, self.num_qk_heads, self.key_dim, self.value_dim
        C = self.channels
        state = cache.state.view(cache.state.shape[0], -1)
        raw = linear_float32_out(x, self.gate_rows)
        proj = linear(x, self.in_weight, next_weight=self.o_weight)
        conv = torch.empty((T, C), device=x.device, dtype=torch.float32)
        ops.causal_conv(proj[:, :C], self.conv_weight, None, state[:, self.memory_floats:] if self.taps > 1 else None, step.state_slots,
                        step.cu_seqlens_q, step.seq_index, step.num_seqs, conv, activation="silu")
        o = torch.empty((T, self.v_width), device=x.device, dtype=torch.float32)
        ops.delta_scan(conv, 0, self.qk_width, 2 * self.qk_width, raw, self.a_log, self.dt_bias, state, step.state_slots, step.cu_seqlens_q, o,
                       step.num_seqs, H, G, d, e, self.q_scale, self.unit_eps)
        y = torch.empty((T, self.v_width), device=x.device, dtype=x.dtype)
        ops.gla_norm_gate(o, proj[:, C:], self.norm_weight, y, H, e, self.norm_eps)
        return linear(y, self.o_weight, next_weight=step.weight_after)
