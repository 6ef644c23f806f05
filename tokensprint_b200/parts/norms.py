"""RMSNorm over the float32 residual stream, fused with the residual sum before it."""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from tokensprint_b200 import ops
from tokensprint_b200.parts.base import NormParams, BuildContext, Norm, TensorSpec, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    """y = x * rsqrt(mean(x^2) + eps) * (offset + weight), no bias.  `offset` 0 (the default): a plain
    weight; 1: a weight that is stored as its distance from one.  The sum offset + weight is
    taken once, in float32, when the weight is loaded.

    Reference: engine/nn/base_layers.py:38-46 and engine/kernels/triton/rmsnorm.py:19-42.
    """

    graph_safe = True
    reads_through_ops = True

    def __init__(self, ctx: BuildContext, *, dim: int, eps: float, weight: str, offset: float = 0.0, scalar: bool = False) -> None:
        self.dim, self.eps, self.weight_name, self.offset = int(dim), float(eps), weight, float(offset)
        self.scalar = bool(scalar)
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.weight_name, () if self.scalar else (self.dim,), "vector")]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name]
        if self.scalar:
            self.weight = self.weight.reshape(1).expand(self.dim).contiguous()
        if self.offset:
            self.weight = (self.weight + self.offset).contiguous()

    def params(self) -> Optional[NormParams]:
        return NormParams(self.weight, self.eps, self.dim)

    def forward(self, hidden, delta, out, row_index=None) -> None:
        ops.add_rmsnorm(hidden, delta, self.weight, out, self.eps, row_index)

    def forward_branch(self, branch, hidden, rounded=None) -> None:
        ops.rmsnorm_add(branch, self.weight, hidden, self.eps, rounded)
