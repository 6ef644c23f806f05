"""Several mixers side by side on the same input, their outputs added with fixed weights."""

from __future__ import annotations

from typing import Mapping, Optional, Sequence

import torch

from tokensprint_b200 import ops
from tokensprint_b200.parts.base import BuildContext, CacheNeed, LayerCache, Mixer, PartSpec, StepContext, TensorSpec, build_part, register_part


@register_part("mixer", "parallel")
class ParallelMixers(Mixer):
    """y = sum_i scale_i * mixer_i(x): `mixers` is a list of mixer specs, `scales` one number each.

    The branches share the run's cache: at most one of them may page keys and values and at most
    one may keep a state slot (a softmax attention beside a recurrent mixer, say); each is handed
    the part of the `LayerCache` it asked for."""

    def __init__(self, ctx: BuildContext, *, mixers: Sequence[PartSpec], scales: Sequence[float]) -> None:
        if not mixers or len(mixers) != len(scales) or len(mixers) > ops.WEIGHTED_SUM_MAX_INPUTS:
            raise ValueError(f"parallel mixers: one scale per mixer, one to {ops.WEIGHTED_SUM_MAX_INPUTS} mixers")
        self.mixers = [build_part("mixer", m, ctx) for m in mixers]
        self.scales = [float(s) for s in scales]
        needs = [m.cache_need() for m in self.mixers]
        self._paged = [i for i, n in enumerate(needs) if n.kind != "none"]
        self._stateful = [i for i, n in enumerate(needs) if n.state_shape is not None]
        if len(self._paged) > 1 or len(self._stateful) > 1:
            raise ValueError("parallel mixers: at most one branch with pages and one with a state slot")
        self._needs = needs
        self.graph_safe = all(m.graph_safe for m in self.mixers)
        self.reads_through_ops = all(m.reads_through_ops for m in self.mixers)

    def first_weight(self) -> Optional[torch.Tensor]:
        return self.mixers[0].first_weight()

    def cache_need(self) -> CacheNeed:
        paged = self._needs[self._paged[0]] if self._paged else CacheNeed()
        st = self._needs[self._stateful[0]] if self._stateful else CacheNeed()
        if paged.kind == "none":
            return CacheNeed(kind="none", state_shape=st.state_shape, state_dtype=st.state_dtype)
        return CacheNeed(kind=paged.kind, window=paged.window, k_row=paged.k_row, v_row=paged.v_row, single_pool=paged.single_pool,
                         state_shape=st.state_shape, state_dtype=st.state_dtype)

    def tensor_specs(self) -> list[TensorSpec]:
        return [s for m in self.mixers for s in m.tensor_specs()]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for m in self.mixers:
            m.load(tensors)

    def forward(self, x: torch.Tensor, step: StepContext, cache: LayerCache) -> torch.Tensor:
        after = step.weight_after
        outs = []
        for i, m in enumerate(self.mixers):
            if not m.reads_through_ops:
                ops.flush_gemm_chain()
            paged, stateful = i in self._paged, i in self._stateful
            part = LayerCache(group=cache.group if paged else -1, k_pages=cache.k_pages if paged else None,
                              v_pages=cache.v_pages if paged else None, state=cache.state if stateful else None, writes=cache.writes)
            step.weight_after = after if i + 1 == len(self.mixers) else self.mixers[i + 1].first_weight()
            outs.append(m.forward(x, step, part))
        step.weight_after = after
        out = torch.empty_like(outs[0])
        ops.weighted_sum(outs, self.scales, out)
        return out
