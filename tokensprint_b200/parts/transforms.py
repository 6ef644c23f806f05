"""Transforms on the embedding rows that the package itself offers."""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from tokensprint_b200 import ops
from tokensprint_b200.parts.base import BuildContext, CacheNeed, LayerCache, StepContext, TensorSpec, Transform, register_part


@register_part("transform", "pair_hash_embedding")
class PairHashEmbedding(Transform):
    """Adds to every token's embedding row a row of a second table, picked by a hash of the token
    before it and the token itself:  x[t] += table[(id[t-1] * mul_prev + id[t] * mul_cur) mod buckets];
    the first token of a sequence takes the table's last row (index `buckets`).

    The token before a step's first token of a request was part of an earlier step: one int32 word
    per request (a state slot) keeps the last token a request has run, also when that token never
    reached the host (ids fed on the device)."""

    graph_safe = True
    reads_through_ops = True

    def __init__(self, ctx: BuildContext, *, table: str, buckets: int, mul_prev: int, mul_cur: int, hidden_size: int, vocab_size: int) -> None:
        self.name, self.buckets, self.mul_prev, self.mul_cur = table, int(buckets), int(mul_prev), int(mul_cur)
        self.hidden_size, self.vocab_size = int(hidden_size), int(vocab_size)
        if self.buckets < 1 or self.mul_prev < 0 or self.mul_cur < 0:
            raise ValueError("pair_hash_embedding: buckets must be positive and the multipliers not negative")
        self.table: Optional[torch.Tensor] = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name, (self.buckets + 1, self.hidden_size))]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.table = tensors[self.name]

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="none", state_shape=(1,), state_dtype=torch.int32)

    def forward(self, x: torch.Tensor, step: Optional[StepContext], cache: Optional[LayerCache] = None) -> torch.Tensor:
        if step is None or cache is None or cache.state is None:
            raise ops.KernelError("pair_hash_embedding: needs the step's context and its state slots")
        ops.pair_hash_embed(x, self.table, step.token_ids, step.positions, step.seq_index, step.cu_seqlens_q, step.state_slots,
                            cache.state.view(-1), self.buckets, self.mul_prev, self.mul_cur, self.vocab_size)
        return x


@register_part("transform", "pass_entry")
class PassEntry(Transform):
    """What a model adds to the residual stream where a stretch of layers begins (a model that runs
    a stretch several times names one of these before each pass):

        x += embedding rows   (with `add_embedding`: the rows as they entered the first block)
        x += table[row]       (one learned vector of the [rows, width] tensor `table` per pass)

    both in float32, in one kernel."""

    graph_safe = True
    reads_through_ops = True

    def __init__(self, ctx: BuildContext, *, table: Optional[str], rows: int, row: int, hidden_size: int, add_embedding: bool) -> None:
        self.name, self.rows, self.row, self.hidden_size = table, int(rows), int(row), int(hidden_size)
        self.add_embedding = bool(add_embedding)
        if table is not None and not 0 <= self.row < self.rows:
            raise ValueError(f"pass_entry: row {row} of a table of {rows} rows")
        self.vector: Optional[torch.Tensor] = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [] if self.name is None else [TensorSpec(self.name, (self.rows, self.hidden_size), "vector")]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        if self.name is not None:
            keep = getattr(tensors, "keep", None)  # one copy of the table for all passes
            table = keep(self.name) if keep is not None else tensors[self.name]
            self.vector = table[self.row]

    def forward(self, x: torch.Tensor, step: Optional[StepContext], embedding: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.add_embedding and embedding is None:
            raise ops.KernelError("pass_entry: the embedding rows were not kept for this step")
        ops.stream_add(x, embedding if self.add_embedding else None, self.vector)
        return x


@register_part("transform", "scale")
class Scale(Transform):
    """x <- factor * x in float32: a constant on the logits (or on the embedding rows)."""

    graph_safe = True
    reads_through_ops = True

    def __init__(self, ctx: BuildContext, *, factor: float) -> None:
        self.factor = float(factor)

    def forward(self, x: torch.Tensor, step: Optional[StepContext]) -> torch.Tensor:
        ops.scale_rows(x, self.factor)
        return x


@register_part("transform", "softcap")
class SoftCap(Transform):
    """x <- cap * tanh(x / cap) in float32: logits bent smoothly into (-cap, cap)."""

    graph_safe = True
    reads_through_ops = True

    def __init__(self, ctx: BuildContext, *, cap: float) -> None:
        self.cap = float(cap)
        if not self.cap > 0:
            raise ValueError("softcap: the cap must be positive")

    def forward(self, x: torch.Tensor, step: Optional[StepContext]) -> torch.Tensor:
        ops.softcap_rows(x, self.cap)
        return x
