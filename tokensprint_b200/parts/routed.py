"""Feed-forward layers beside SwiGLU: a plain two-matrix layer with an activation, a gated layer
with capped operands, a layer of routed experts of that form, and a per-layer token input."""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from tokensprint_b200 import ops
from tokensprint_b200.parts.base import BuildContext, FeedForward, PartSpec, StepContext, TensorSpec, build_part, register_part
from tokensprint_b200.parts.linear import linear

ACTIVATIONS = {"gelu_tanh": ops.gelu_tanh}


@register_part("feed_forward", "activated")
class ActivatedFeedForward(FeedForward):
    """f = W_down act(W_up x), no biases; `activation`: "gelu_tanh"."""

    graph_safe = True
    reads_through_ops = True

    def __init__(self, ctx: BuildContext, *, hidden_size: int, intermediate_size: int, up: str, down: str, activation: str = "gelu_tanh") -> None:
        if activation not in ACTIVATIONS:
            raise ValueError(f"activated feed-forward: unknown activation {activation!r}; known: {sorted(ACTIVATIONS)}")
        self.hidden_size, self.intermediate_size, self.activation = int(hidden_size), int(intermediate_size), activation
        self.names = {"up": up, "down": down}
        self.up: Optional[torch.Tensor] = None
        self.down: Optional[torch.Tensor] = None

    def first_weight(self) -> Optional[torch.Tensor]:
        return self.up

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.names["up"], (self.intermediate_size, self.hidden_size)),
                TensorSpec(self.names["down"], (self.hidden_size, self.intermediate_size))]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.up, self.down = tensors[self.names["up"]], tensors[self.names["down"]]

    def forward(self, x: torch.Tensor, step: StepContext) -> torch.Tensor:
        h = linear(x, self.up, next_weight=self.down)
        ACTIVATIONS[self.activation](h, h)
        return linear(h, self.down, next_weight=step.weight_after if step is not None else None)


@register_part("feed_forward", "capped_glu")
class CappedGLUFeedForward(FeedForward):
    """f = W_down (a * sigmoid(alpha a) * (b + 1)) with a = min(W_gate x, limit) and
    b = clamp(W_up x, -limit, limit); no biases.  Gate and up are stacked into one product."""

    graph_safe = True
    reads_through_ops = True

    def __init__(self, ctx: BuildContext, *, hidden_size: int, intermediate_size: int, gate: str, up: str, down: str, limit: float,
                 alpha: float = 1.702) -> None:
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.limit, self.alpha = float(limit), float(alpha)
        self.names = {"gate": gate, "up": up, "down": down}
        self.gate_up: Optional[torch.Tensor] = None
        self.down: Optional[torch.Tensor] = None

    def first_weight(self) -> Optional[torch.Tensor]:
        return self.gate_up

    def tensor_specs(self) -> list[TensorSpec]:
        H, I = self.hidden_size, self.intermediate_size
        return [TensorSpec(self.names["gate"], (I, H)), TensorSpec(self.names["up"], (I, H)), TensorSpec(self.names["down"], (H, I))]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.gate_up = torch.cat([tensors[self.names["gate"]], tensors[self.names["up"]]], dim=0).contiguous()
        self.down = tensors[self.names["down"]]

    def forward(self, x: torch.Tensor, step: StepContext) -> torch.Tensor:
        gu = linear(x, self.gate_up, next_weight=self.down)
        act = torch.empty((x.shape[0], self.intermediate_size), device=x.device, dtype=x.dtype)
        ops.capped_glu(gu, act, self.limit, self.alpha)
        return linear(act, self.down)


@register_part("feed_forward", "routed_experts")
class RoutedExperts(FeedForward):
    """`num_experts` gated experts of which each token uses `top`:

        z = W_router x (+ b, if `router_bias` names one)   (float32; from the float32 residual rows
                                                            where the block has them)
        chosen = the `top` largest logits
        weights: `score` "sigmoid": w_e = sigmoid(z_e) (or that / their sum with `renormalize`);
                 "softmax_chosen": the softmax over the chosen logits alone
                 "softmax_all": scores s = softmax(z) over all experts; the `top` largest of
                 s + c are chosen (`correction` names c, a number per expert that steers the choice
                 only) and the weights are the chosen s themselves (divided by their sum with `renormalize`)
        f = sum over chosen e of expert_e(w_e x)   (`weight_on` "input"; "output": w_e expert_e(x))
            + shared(x) if a shared expert is named (any feed-forward spec)
        expert(x) = W_down act(W_gate x, W_up x), `activation` "capped_glu" (with `limit`, `alpha`)
                    or "swiglu" (silu(gate) * up); "gelu": experts without a gate matrix,
                    W_down gelu(W_up x) with the exact (erf) gelu
        `identity` = n: the router has n more outputs than there are experts; the last n stand for
                    identity experts, which have no tensors and whose output is their input x itself
                    (times the weight; `weight_on` "output" only)

    Routing, the sort of the (token, choice) pairs by expert and both expert products run on the
    device with grids that depend on the token count only, so a decode step is a fixed kernel
    sequence.  The experts' matrices are stacked at load: gate, up [E, I, H], down [E, H, I].
    """

    graph_safe = True
    wants_residual = True

    def __init__(self, ctx: BuildContext, *, hidden_size: int, num_experts: int, top: int, intermediate_size: int,
                 router: str, expert_prefix: str, limit: float = 0.0, alpha: float = 1.702, renormalize: bool = False,
                 weight_on: str = "input", shared: Optional[PartSpec] = None, router_bias: Optional[str] = None,
                 score: str = "sigmoid", activation: str = "capped_glu", correction: Optional[str] = None, identity: int = 0) -> None:
        self.hidden_size, self.num_experts, self.top = int(hidden_size), int(num_experts), int(top)
        self.intermediate_size, self.limit, self.alpha = int(intermediate_size), float(limit), float(alpha)
        self.renormalize = bool(renormalize)
        if not 0 < self.top:
            raise ValueError(f"routed experts: top {top} of {num_experts} experts")
        if weight_on not in ("input", "output"):
            raise ValueError(f"routed experts: weight_on must be 'input' or 'output', got {weight_on!r}")
        if score not in ops.ROUTER_SCORES:
            raise ValueError(f"routed experts: score must be one of {sorted(ops.ROUTER_SCORES)}, got {score!r}")
        if activation not in ops.MOE_ACTIVATIONS:
            raise ValueError(f"routed experts: activation must be one of {sorted(ops.MOE_ACTIVATIONS)}, got {activation!r}")
        self.weight_on, self.score, self.activation = weight_on, score, activation
        self.identity = int(identity)
        if self.identity < 0 or (self.identity and weight_on != "output"):
            raise ValueError("routed experts: identity experts hand on their input times the weight (weight_on = 'output')")
        if self.top > self.num_experts + self.identity:
            raise ValueError(f"routed experts: top {top} of {num_experts} + {identity} router outputs")
        if correction is not None and score != "softmax_all":
            raise ValueError("routed experts: a correction of the choice comes with score = 'softmax_all'")
        self.gated = activation != "gelu"
        self.correction_name = correction
        self.correction: Optional[torch.Tensor] = None
        self.router_name, self.router_bias_name, self.prefix = router, router_bias, expert_prefix
        self.router_bias: Optional[torch.Tensor] = None
        self.shared = build_part("feed_forward", shared, ctx) if shared is not None else None
        if self.shared is not None:
            self.graph_safe = self.shared.graph_safe
        self.reads_through_ops = self.shared is None or self.shared.reads_through_ops
        self.dtype = ctx.dtype

    def first_weight(self) -> Optional[torch.Tensor]:
        return None

    def _expert_names(self, e: int) -> tuple[str, str, str]:
        p = f"{self.prefix}{e}."
        return p + "gate", p + "up", p + "down"

    def tensor_specs(self) -> list[TensorSpec]:
        H, I = self.hidden_size, self.intermediate_size
        outputs = self.num_experts + self.identity
        specs = [TensorSpec(self.router_name, (outputs, H), "vector")]  # the router stays float32
        if self.router_bias_name is not None:
            specs.append(TensorSpec(self.router_bias_name, (outputs,), "vector"))
        if self.correction_name is not None:
            specs.append(TensorSpec(self.correction_name, (outputs,), "vector"))
        for e in range(self.num_experts):
            g, u, d = self._expert_names(e)
            specs += ([TensorSpec(g, (I, H))] if self.gated else []) + [TensorSpec(u, (I, H)), TensorSpec(d, (H, I))]
        if self.shared is not None:
            specs += self.shared.tensor_specs()
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.router = tensors[self.router_name]
        if self.router_bias_name is not None:
            self.router_bias = tensors[self.router_bias_name]
        if self.correction_name is not None:
            self.correction = tensors[self.correction_name]
        names = [self._expert_names(e) for e in range(self.num_experts)]
        self.gate = torch.stack([tensors[g] for g, _, _ in names]).contiguous() if self.gated else None
        self.up = torch.stack([tensors[u] for _, u, _ in names]).contiguous()
        self.down = torch.stack([tensors[d] for _, _, d in names]).contiguous()
        if self.shared is not None:
            self.shared.load(tensors)

    def forward(self, x: torch.Tensor, step: StepContext, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        T, top, dev = x.shape[0], self.top, x.device
        rows = residual if residual is not None else x  # float32 rows where the block has them, else their rounding
        chosen = torch.empty((T, top), device=dev, dtype=torch.int32)
        weights = torch.empty((T, top), device=dev, dtype=torch.float32)
        ops.router(rows, self.router, top, self.renormalize, chosen, weights, bias=self.router_bias, score=self.score, correction=self.correction)
        # both products take the same plan: the tensor cores only if both inner widths suit them
        tensor_cores = ops.moe_on_tensor_cores(x.dtype, self.hidden_size, self.intermediate_size)
        plan = ops.moe_plan(chosen, self.num_experts, ops.moe_row_tile(tensor_cores, T * top, self.num_experts))
        act = torch.empty((T * top, self.intermediate_size), device=dev, dtype=x.dtype)
        on_input = self.weight_on == "input"
        ones = None if on_input else torch.ones((T * top,), device=dev, dtype=torch.float32)
        ops.moe_gate_up(x, weights.view(-1) if on_input else ones, plan, self.gate, self.up, act, top, self.limit, self.alpha,
                        activation=self.activation)
        pair_out = torch.empty((T * top, self.hidden_size), device=dev, dtype=x.dtype)
        ops.moe_down(act, plan, self.down, pair_out)
        shared = None
        if self.shared is not None:
            if not self.shared.reads_through_ops:
                ops.flush_gemm_chain()
            shared = self.shared.forward(x, step)
        out = torch.empty((T, self.hidden_size), device=dev, dtype=x.dtype)
        if self.identity:  # pairs that chose an identity expert have no place in the plan: the combine reads x for them
            ops.moe_combine(pair_out, shared, out, top, weights.view(-1), ids=chosen, num_experts=self.num_experts, x=x)
        else:
            ops.moe_combine(pair_out, shared, out, top, None if on_input else weights.view(-1))
        return out


@register_part("feed_forward", "token_gated_input")
class TokenGatedInput(FeedForward):
    """A per-layer input from a second token table: with e = table[token][column0 : column0 + dim]
    (this layer's slice of the token's row), f = W_proj (act(W_gate x) * e).  The table is shared by
    all layers that name it."""

    graph_safe = True
    reads_through_ops = True

    def __init__(self, ctx: BuildContext, *, hidden_size: int, dim: int, table: str, table_width: int, column0: int, vocab_size: int,
                 gate: str, proj: str) -> None:
        self.hidden_size, self.dim, self.table_width, self.column0 = int(hidden_size), int(dim), int(table_width), int(column0)
        self.vocab_size = int(vocab_size)
        if self.column0 < 0 or self.column0 + self.dim > self.table_width:
            raise ValueError("token gated input: the slice does not fit the table's rows")
        self.names = {"table": table, "gate": gate, "proj": proj}

    def first_weight(self) -> Optional[torch.Tensor]:
        return None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.names["table"], (self.vocab_size, self.table_width)),
                TensorSpec(self.names["gate"], (self.dim, self.hidden_size)),
                TensorSpec(self.names["proj"], (self.hidden_size, self.dim))]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        keep = getattr(tensors, "keep", None)  # one copy of the table for all layers
        self.table = keep(self.names["table"]) if keep is not None else tensors[self.names["table"]]
        self.gate, self.proj = tensors[self.names["gate"]], tensors[self.names["proj"]]

    def forward(self, x: torch.Tensor, step: StepContext) -> torch.Tensor:
        g = linear(x, self.gate)
        ops.gelu_gate_rows(g, self.table, step.token_ids, self.column0)
        return linear(g, self.proj)
