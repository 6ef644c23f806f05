"""A selective state-space layer with one decay per head (Mamba-2) as a mixer part: its state and
the last inputs of its short convolution per request live in a float32 state slot of the cache."""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from tokensprint_b200 import ops
from tokensprint_b200.parts.base import BuildContext, CacheNeed, LayerCache, Mixer, StepContext, TensorSpec, register_part
from tokensprint_b200.parts.linear import linear, linear_float32_out


@register_part("mixer", "state_space")
class StateSpace(Mixer):
    """With H heads of e value channels (inner = H e), state width N and G groups of B and C:

        [z | x | B | C | dt] = W_in h            inner, inner, G N, G N, H columns
        [x | B | C] <- silu(conv(...))           causal, per channel, `taps` wide, with a bias
        dt <- softplus(dt + dt_bias)
        S_t = exp(-exp(A_log_h) dt) S_(t-1) + dt B_t x_t^T      per head, S [N, e]; head h reads group h // (H / G)
        y_t = S_t^T C_t + D_h x_t
        out = W_o ( norm_in_parts(y * silu(z)) * w_norm )       the row in `norm_groups` equal parts, each by its own rms

    Parameters: `hidden_size`, `num_heads`, `value_dim`, `state_dim`, `groups`, `taps`, `norm_groups`,
    `norm_eps` and the tensors' names.  The step-size rows of W_in are a product of their own whose
    sums leave in float32 (never rounded to the compute dtype); the convolution, the step sizes, decays, the state, the recurrence and the norm are
    float32 whatever the compute dtype.  The state slot holds [H, N, e] followed by the last taps - 1
    inputs of the convolution [taps - 1, inner + 2 G N], oldest first; zeros before the first token."""

    graph_safe = True
    reads_through_ops = True

    def __init__(self, ctx: BuildContext, *, hidden_size: int, num_heads: int, value_dim: int, state_dim: int, groups: int, taps: int,
                 norm_groups: int, norm_eps: float, in_proj: str, conv: str, conv_bias: str, dt_bias: str, a_log: str, skip: str, norm: str,
                 o: str) -> None:
        self.hidden_size, self.num_heads, self.value_dim = int(hidden_size), int(num_heads), int(value_dim)
        self.state_dim, self.groups, self.taps, self.norm_groups = int(state_dim), int(groups), int(taps), int(norm_groups)
        self.norm_eps = float(norm_eps)
        if min(self.num_heads, self.value_dim, self.state_dim, self.groups, self.taps, self.norm_groups) < 1:
            raise ValueError("state space: every size must be positive")
        if self.num_heads % self.groups or (self.num_heads * self.value_dim) % self.norm_groups:
            raise ValueError("state space: heads must be a multiple of groups, and heads * value_dim of norm_groups")
        if self.state_dim > ops.GLA_MAX_KEY_DIM:
            raise ValueError(f"state space: state_dim {state_dim} exceeds the kernel's {ops.GLA_MAX_KEY_DIM}")
        self.inner = self.num_heads * self.value_dim
        self.channels = self.inner + 2 * self.groups * self.state_dim
        self.memory_floats = self.num_heads * self.state_dim * self.value_dim
        self.names = {"in": in_proj, "conv": conv, "conv_bias": conv_bias, "dt_bias": dt_bias, "a_log": a_log, "skip": skip, "norm": norm, "o": o}
        self.in_weight: Optional[torch.Tensor] = None  # the rows of z, x, B, C
        self.dt_weight: Optional[torch.Tensor] = None  # the step-size rows
        self.o_weight: Optional[torch.Tensor] = None

    def first_weight(self) -> Optional[torch.Tensor]:
        return self.in_weight

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="none", state_shape=(self.memory_floats + (self.taps - 1) * self.channels,), state_dtype=torch.float32)

    def tensor_specs(self) -> list[TensorSpec]:
        W, n, H = self.hidden_size, self.names, self.num_heads
        return [TensorSpec(n["in"], (self.inner + self.channels + H, W)), TensorSpec(n["conv"], (self.channels, self.taps), "vector"),
                TensorSpec(n["conv_bias"], (self.channels,), "vector"), TensorSpec(n["dt_bias"], (H,), "vector"),
                TensorSpec(n["a_log"], (H,), "vector"), TensorSpec(n["skip"], (H,), "vector"), TensorSpec(n["norm"], (self.inner,), "vector"),
                TensorSpec(n["o"], (W, self.inner))]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        w = tensors[n["in"]]
        rows = self.inner + self.channels
        self.in_weight = w[:rows].contiguous()
        self.dt_weight = w[rows:].contiguous()
        self.conv_weight, self.conv_bias = tensors[n["conv"]], tensors[n["conv_bias"]]
        self.dt_bias, self.a_log, self.skip = tensors[n["dt_bias"]], tensors[n["a_log"]], tensors[n["skip"]]
        self.norm_weight, self.o_weight = tensors[n["norm"]], tensors[n["o"]]

    def forward(self, x: torch.Tensor, step: StepContext, cache: LayerCache) -> torch.Tensor:
        if cache.state is None:
            raise ops.KernelError("state space: this mixer needs a state slot per request (none was bound to its run)")
        if not cache.writes:
            raise ops.KernelError("state space: a run cannot read another run's state")
        T, H, e, N, G = x.shape[0], self.num_heads, self.value_dim, self.state_dim, self.groups
        inner, GN = self.inner, self.groups * self.state_dim
        state = cache.state.view(cache.state.shape[0], -1)
        dt_raw = linear_float32_out(x, self.dt_weight)
        proj = linear(x, self.in_weight, next_weight=self.o_weight)
        z = proj[:, :inner]
        conv, dt, decay = ops.ssm_conv(proj[:, inner:], self.conv_weight, self.conv_bias, state[:, self.memory_floats:], step.state_slots,
                                       step.cu_seqlens_q, step.seq_index, step.num_seqs, dt_raw, self.dt_bias, self.a_log)
        xs, Bs, Cs = conv[:, :inner], conv[:, inner:inner + GN], conv[:, inner + GN:]
        o = torch.empty((T, inner), device=x.device, dtype=torch.float32)
        ops.linear_scan(Cs, Bs, xs, decay, dt, 1.0, state, step.state_slots, step.cu_seqlens_q, o, step.num_seqs, H, G, N, e,
                        max_seqlen=step.max_seqlen_q)
        y = torch.empty((T, inner), device=x.device, dtype=x.dtype)
        ops.ssm_gate_norm(o, xs, self.skip, z, self.norm_weight, y, H, e, self.norm_groups, self.norm_eps)
        return linear(y, self.o_weight, next_weight=step.weight_after)
