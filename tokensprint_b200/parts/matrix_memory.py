"""A matrix memory with exponential gates (the mLSTM cell of xLSTM) as a mixer part: its memory,
normaliser and running maximum per request live in a float32 state slot of the cache."""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from tokensprint_b200 import ops
from tokensprint_b200.parts.base import BuildContext, CacheNeed, LayerCache, Mixer, StepContext, TensorSpec, register_part
from tokensprint_b200.parts.linear import linear, linear_float32_out


@register_part("mixer", "matrix_memory")
class MatrixMemory(Mixer):
    """Per head, with key width d and value width e, for the tokens of a sequence in order:

        q_t = W_q x_t * q_scale,  k_t = W_k x_t,  v_t = W_v x_t
        log_i = cap tanh((W_i x_t + b_i) / cap),  log_f = logsigmoid(cap tanh((W_f x_t + b_f) / cap))
        m_t = max(log_f + m_(t-1), log_i)                                   m = 0 before the first token
        S_t = exp(log_f + m_(t-1) - m_t) S_(t-1) + exp(log_i - m_t) k_t v_t^T   S [d, e], n [d] likewise with k_t alone
        o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
        y_t = W_o ( concat over heads of  o_t / rms(o_t) ) * w_norm * sigmoid(W_g x_t)

    Parameters: `hidden_size`, `num_heads`, `key_dim`, `value_dim`, `gate_cap`, `norm_eps`, `q_scale`
    (default key_dim^-0.5) and the tensors' names.  q, k, v and the output gate come from one stacked
    product in the compute dtype; the two gates' pre-activations from a product of their own whose
    sums leave in float32 (never rounded to the compute dtype); their biases, the tanh caps, gates,
    running maximum, memory, normaliser, read-out and head norm are float32 whatever the compute
    dtype.  The state slot holds [heads, d, e + 1] (memory with the normaliser as a last column)
    followed by [heads] running maxima; it is carried from step to step, so prompts may be cut anywhere."""

    graph_safe = True
    reads_through_ops = True

    def __init__(self, ctx: BuildContext, *, hidden_size: int, num_heads: int, key_dim: int, value_dim: int, gate_cap: float, norm_eps: float,
                 q: str, k: str, v: str, gate: str, o: str, norm: str, input_gate: str, input_gate_bias: str, forget_gate: str,
                 forget_gate_bias: str, q_scale: Optional[float] = None) -> None:
        self.hidden_size, self.num_heads, self.key_dim, self.value_dim = int(hidden_size), int(num_heads), int(key_dim), int(value_dim)
        self.gate_cap, self.norm_eps = float(gate_cap), float(norm_eps)
        if min(self.num_heads, self.key_dim, self.value_dim) < 1 or not self.gate_cap > 0:
            raise ValueError("matrix memory: heads, key_dim, value_dim and gate_cap must be positive")
        if self.key_dim > ops.GLA_MAX_KEY_DIM:
            raise ValueError(f"matrix memory: key_dim {key_dim} exceeds the kernel's {ops.GLA_MAX_KEY_DIM}")
        self.q_scale = float(q_scale) if q_scale is not None else float(self.key_dim) ** -0.5
        self.names = {"q": q, "k": k, "v": v, "gate": gate, "o": o, "norm": norm, "i": input_gate, "i_bias": input_gate_bias,
                      "f": forget_gate, "f_bias": forget_gate_bias}
        self.memory_floats = self.num_heads * self.key_dim * (self.value_dim + 1)
        self.in_weight: Optional[torch.Tensor] = None  # [q | k | v | gate] stacked
        self.gates_weight: Optional[torch.Tensor] = None  # [input-gate rows ; forget-gate rows]
        self.gates_bias: Optional[torch.Tensor] = None
        self.norm_weight: Optional[torch.Tensor] = None
        self.o_weight: Optional[torch.Tensor] = None

    def first_weight(self) -> Optional[torch.Tensor]:
        return self.in_weight

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="none", state_shape=(self.memory_floats + self.num_heads,), state_dtype=torch.float32)

    def tensor_specs(self) -> list[TensorSpec]:
        W, n, H = self.hidden_size, self.names, self.num_heads
        hd, he = H * self.key_dim, H * self.value_dim
        return [TensorSpec(n["q"], (hd, W)), TensorSpec(n["k"], (hd, W)), TensorSpec(n["v"], (he, W)), TensorSpec(n["gate"], (he, W)),
                TensorSpec(n["o"], (W, he)), TensorSpec(n["norm"], (he,), "vector"), TensorSpec(n["i"], (H, W)),
                TensorSpec(n["i_bias"], (H,), "vector"), TensorSpec(n["f"], (H, W)), TensorSpec(n["f_bias"], (H,), "vector")]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        self.in_weight = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]], tensors[n["gate"]]], dim=0).contiguous()
        self.gates_weight = torch.cat([tensors[n["i"]], tensors[n["f"]]], dim=0).contiguous()
        self.gates_bias = torch.cat([tensors[n["i_bias"]], tensors[n["f_bias"]]], dim=0).contiguous()
        self.norm_weight, self.o_weight = tensors[n["norm"]], tensors[n["o"]]

    def forward(self, x: torch.Tensor, step: StepContext, cache: LayerCache) -> torch.Tensor:
        if cache.state is None:
            raise ops.KernelError("matrix memory: this mixer needs a state slot per request (none was bound to its run)")
        if not cache.writes:
            raise ops.KernelError("matrix memory: a run cannot read another run's state")
        T, H, d, e = x.shape[0], self.num_heads, self.key_dim, self.value_dim
        hd, he = H * d, H * e
        state = cache.state.view(cache.state.shape[0], -1)
        pre = linear_float32_out(x, self.gates_weight)
        decay, kscale, m = ops.mlstm_gate_scan(pre, self.gate_cap, state[:, self.memory_floats:], step.state_slots, step.cu_seqlens_q,
                                               step.num_seqs, H, bias=self.gates_bias)
        proj = linear(x, self.in_weight, next_weight=self.o_weight)
        q, k, v, gate = proj[:, :hd], proj[:, hd:2 * hd], proj[:, 2 * hd:2 * hd + he], proj[:, 2 * hd + he:]
        o = torch.empty((T, H * (e + 1)), device=x.device, dtype=torch.float32)
        ops.linear_scan(q, k, v, decay, kscale, self.q_scale, state, step.state_slots, step.cu_seqlens_q, o, step.num_seqs, H, H, d, e,
                        normaliser=True, max_seqlen=step.max_seqlen_q)
        y = torch.empty((T, he), device=x.device, dtype=x.dtype)
        ops.mlstm_norm_gate(o, m, gate, self.norm_weight, y, H, e, self.norm_eps)
        return linear(y, self.o_weight, next_weight=step.weight_after)
