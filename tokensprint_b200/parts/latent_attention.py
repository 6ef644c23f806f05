"""Latent attention over the paged cache, as a mixer part: per token the cache holds one low-rank
latent row and one rotated key part, shared by all heads."""

from __future__ import annotations

import os
from typing import Mapping, Optional

import torch

from tokensprint_b200 import ops
from tokensprint_b200.parts.base import BuildContext, CacheNeed, LayerCache, Mixer, PartSpec, StepContext, TensorSpec, build_part, register_part
from tokensprint_b200.parts.linear import linear, linear_float32_out


# TS_LATENT_ATTENTION_MMA=0 (for measurements): bfloat16 steps also run the CUDA-core kernel.
LATENT_ATTENTION_MMA = os.environ.get("TS_LATENT_ATTENTION_MMA", "1") != "0"
# Up to this many tokens per sequence a step's keys are cut into ranges (decode, and the shortest portions).
LATENT_DECODE_MAX_TOKENS = 4


def batched_linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[b] = a[b] @ w[b]^T for a batch of small products (one per head): float32 through the
    engine's FFMA kernel, bfloat16 through the library's batched GEMM."""
    if a.dtype == torch.float32:
        ops.sgemm_nt_batched(a, w, out)
    else:
        ops.library_bmm(a, w, out)


@register_part("mixer", "latent_attention")
class LatentAttentionMixer(Mixer):
    """Attention whose keys and values are rebuilt from a latent:

        q_a = [q_plain,a ; q_rot,a]          H heads of nope_dim + rot_dim query entries
        [c ; r] = W_dkv x                    c: kv_rank entries, RMS-normed; r: rot_dim entries, rotated
        k_a = [U_k,a c ; r],  v_a = U_v,a c  (r is the same for every head)
        o_a = softmax(q_a . k_a * scale) v_a, times sigmoid(W_g x)_a if `gate` is named;  y = W_o [o_a]

    Only [c ; r] is cached, one row of kv_rank + rot_dim entries per token in a single pool.  The
    keys are never rebuilt: U_k,a^T q_plain,a (the absorbed query) is scored against c directly,
    the weighted sum runs over c, and U_v,a is applied to that sum.  A step is: one product for
    [q | c, r | gate logits], the prepare kernel (norm, rotation, store), the per-head absorbing
    products, the attention kernel, the per-head value products, the output product.

    `q_rank` > 0: the queries pass a latent of their own first, q = W_uq norm(W_dq x) with an RMS
    norm and weight `dq_norm` over the q_rank entries (`q` then names W_uq [H (nope + rot), q_rank] and
    `dq` names W_dq [q_rank, hidden]); the latent's rows leave their product in float32 for the norm.
    `dkv` None: the layer has no latent of its own; its run reads the rows another layer's run cached
    (same kv_rank, rot_dim and rotation), with its own queries, U_k, U_v and output matrix.
    A rotation whose frequencies are stretched brings a magnitude on its cosines and sines.

    Parameters: sizes (`hidden_size`, `num_heads`, `nope_dim`, `rot_dim`, `value_dim`, `kv_rank`),
    `scale`, `norm_eps` of the latent's norm, `window` (0: all earlier keys), `position` (a rotary
    spec: its width is the number of rotated entries of the rot_dim part, its pairing is honoured)
    and the checkpoint names of the tensors.
    """

    reads_through_ops = False  # the per-head products may be the library's

    def __init__(self, ctx: BuildContext, *, hidden_size: int, num_heads: int, nope_dim: int, rot_dim: int, value_dim: int, kv_rank: int,
                 scale: float, norm_eps: float, q: str, dkv: Optional[str], dkv_norm: Optional[str], uk: str, uv: str, o: str,
                 gate: Optional[str] = None, window: int = 0, position: Optional[PartSpec] = None, q_rank: int = 0, dq: Optional[str] = None,
                 dq_norm: Optional[str] = None) -> None:
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.nope_dim, self.rot_dim, self.value_dim, self.kv_rank = int(nope_dim), int(rot_dim), int(value_dim), int(kv_rank)
        self.scale, self.norm_eps, self.window = float(scale), float(norm_eps), int(window or 0)
        if min(self.num_heads, self.kv_rank, self.value_dim) < 1 or self.nope_dim < 0 or self.rot_dim < 0 or self.nope_dim + self.rot_dim < 1:
            raise ValueError("latent attention: heads, kv_rank and value_dim must be positive, and a head needs query entries")
        self.q_rank = int(q_rank or 0)
        if (self.q_rank > 0) != (dq is not None) or (dq is None) != (dq_norm is None):
            raise ValueError("latent attention: a query latent needs q_rank and the names of its matrix and norm weight")
        if (dkv is None) != (dkv_norm is None):
            raise ValueError("latent attention: the latent's matrix and its norm weight come together")
        self.names = {"q": q, "dkv": dkv, "dkv_norm": dkv_norm, "uk": uk, "uv": uv, "o": o, "gate": gate, "dq": dq, "dq_norm": dq_norm}
        self.position = build_part("position_encoding", position, ctx) if position is not None else None
        self.rot_dims, self.pairing, self.magnitude = 0, "half", 1.0
        if self.position is not None:
            self.rot_dims, self.pairing = int(self.position.dim), self.position.pairing
            self.magnitude = float(getattr(self.position, "magnitude", 1.0))
            if self.rot_dims > self.rot_dim:
                raise ValueError(f"latent attention: {self.rot_dims} rotated entries do not fit a rotated part of {self.rot_dim}")
        self.graph_safe = True
        self.dtype = ctx.dtype
        self.stacked: Optional[torch.Tensor] = None
        self.offsets = (0, 0, 0)

    @property
    def key_dim(self) -> int:
        return self.kv_rank + self.rot_dim

    def first_weight(self) -> Optional[torch.Tensor]:
        return self.stacked

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="window" if self.window > 0 else "full", window=self.window, k_row=(self.key_dim,), single_pool=True)

    def tensor_specs(self) -> list[TensorSpec]:
        W, H, n = self.hidden_size, self.num_heads, self.names
        specs = [
            TensorSpec(n["q"], (H * (self.nope_dim + self.rot_dim), self.q_rank or W)),
            TensorSpec(n["uk"], (H * self.nope_dim, self.kv_rank)),
            TensorSpec(n["uv"], (H * self.value_dim, self.kv_rank)),
            TensorSpec(n["o"], (W, H * self.value_dim)),
        ]
        if n["dkv"] is not None:
            specs += [TensorSpec(n["dkv"], (self.key_dim, W)), TensorSpec(n["dkv_norm"], (self.kv_rank,), "vector")]
        if n["dq"] is not None:
            specs += [TensorSpec(n["dq"], (self.q_rank, W)), TensorSpec(n["dq_norm"], (self.q_rank,), "vector")]
        if n["gate"] is not None:
            specs.append(TensorSpec(n["gate"], (H, W)))
        if self.position is not None:
            specs.extend(self.position.tensor_specs())
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n, H = self.names, self.num_heads
        # one product for what reads x in the compute dtype: [q (without a query latent) | c, r | gate logits]
        parts, at = [], 0
        self.offsets = [0, -1, 0]  # columns of the queries, of [c ; r] (-1: none), of the gate logits
        if n["dq"] is None:
            parts.append(tensors[n["q"]])
            at += parts[-1].shape[0]
        if n["dkv"] is not None:
            self.offsets[1] = at
            parts.append(tensors[n["dkv"]])
            at += self.key_dim
        if n["gate"] is not None:
            self.offsets[2] = at
            parts.append(tensors[n["gate"]])
        self.stacked = torch.cat(parts, dim=0).contiguous() if parts else None
        self.latent_weight = tensors[n["dkv_norm"]] if n["dkv"] is not None else None
        self.dq_weight = self.uq_weight = self.dq_norm_weight = None
        if n["dq"] is not None:
            self.dq_weight, self.dq_norm_weight, self.uq_weight = tensors[n["dq"]], tensors[n["dq_norm"]], tensors[n["q"]]
        # per head: U_k,a^T as a matrix [kv_rank, nope_dim] (out, in) for the absorbing product,
        # U_v,a [value_dim, kv_rank] as it is stored
        self.uk_t = tensors[n["uk"]].view(H, self.nope_dim, self.kv_rank).transpose(1, 2).contiguous() if self.nope_dim else None
        self.uv = tensors[n["uv"]].view(H, self.value_dim, self.kv_rank).contiguous()
        self.o_weight = tensors[n["o"]]
        if self.position is not None:
            self.position.load(tensors)

    def forward(self, x: torch.Tensor, step: StepContext, cache: LayerCache) -> torch.Tensor:
        if cache.k_pages is None or cache.group < 0:
            raise ops.KernelError("latent attention: this mixer needs cache pages (none were bound to its run)")
        T, H, R, D = x.shape[0], self.num_heads, self.kv_rank, self.key_dim
        tables = step.groups[cache.group]
        has_latent = self.names["dkv"] is not None
        if has_latent != cache.writes:
            raise ops.KernelError("latent attention: a layer with a latent of its own fills its cache, one without reads another run's")
        proj = linear(x, self.stacked) if self.stacked is not None else None
        q_src = None
        if self.dq_weight is not None:
            # the query latent: its rows leave the product in float32, the norm rounds them once
            low = linear_float32_out(x, self.dq_weight)
            normed = torch.empty((T, self.q_rank), device=x.device, dtype=x.dtype)
            ops.add_rmsnorm(low, None, self.dq_norm_weight, normed, self.norm_eps)
            q_src = linear(normed, self.uq_weight)
        q_abs = torch.empty((T, H, D), device=x.device, dtype=x.dtype)
        gates = torch.empty((T, H), device=x.device, dtype=torch.float32) if self.names["gate"] is not None else None
        q_off, kv_off, gate_off = self.offsets
        ops.latent_prepare(
            proj, q_off, kv_off, gate_off, q_abs, cache.k_pages if has_latent else None, tables.slot_mapping if has_latent else None,
            step.positions, self.latent_weight, self.norm_eps, None if self.position is None else self.position.frequencies(),
            self.rot_dims, self.pairing, gates, H, self.nope_dim, self.rot_dim, R, magnitude=self.magnitude, q_src=q_src)
        if self.nope_dim:
            q_rows = q_src if q_src is not None else proj[:, : H * (self.nope_dim + self.rot_dim)]
            q_plain = q_rows.view(T, H, self.nope_dim + self.rot_dim)[:, :, : self.nope_dim]
            batched_linear(q_plain.transpose(0, 1), self.uk_t, q_abs[:, :, :R].transpose(0, 1))
        else:
            q_abs[:, :, :R].zero_()
        latent_out = torch.empty((T, H, R), device=x.device, dtype=x.dtype)
        self._attend(q_abs, latent_out, gates, step, cache, tables)
        heads_out = torch.empty((T, H, self.value_dim), device=x.device, dtype=x.dtype)
        batched_linear(latent_out.transpose(0, 1), self.uv, heads_out.transpose(0, 1))
        return linear(heads_out.view(T, H * self.value_dim), self.o_weight, next_weight=step.weight_after)

    def _attend(self, q_abs, out, gates, step: StepContext, cache: LayerCache, tables) -> None:
        H, R, rot = self.num_heads, self.kv_rank, self.rot_dim
        if q_abs.dtype != torch.bfloat16 or not LATENT_ATTENTION_MMA or not ops.latent_attention_mma_supported(R, rot):
            # float32 runs, and sizes the tensor-core kernel is not made for
            ops.latent_attention_simple(
                q_abs, cache.k_pages, out, gates, step.positions, step.seq_index, tables.block_table, step.page_size, H, R, rot,
                self.scale, self.window)
            return
        B, singles = step.num_seqs, step.decode_seqs

        def run(first: int, count: int, t0: int, t1: int, max_q: int, split: bool) -> None:
            splits = 1
            if split:
                context = ops.attention_decode_plan_context(step.max_context_len, self.window)
                splits = ops.latent_attention_splits(q_abs.device, count, max_q * H, context, R, rot)
            ops.latent_attention_mma(
                q_abs[t0:t1], cache.k_pages, out[t0:t1], None if gates is None else gates[t0:t1], step.cu_seqlens_q[first : first + count + 1],
                step.context_lens[first : first + count], tables.block_table[first : first + count], step.page_size, count, max_q, H, R, rot,
                self.scale, self.window, splits)

        T = q_abs.shape[0]
        if step.max_seqlen_q <= LATENT_DECODE_MAX_TOKENS:
            run(0, B, 0, T, step.max_seqlen_q, True)  # few rows per sequence: the keys are spread over CTAs
        elif 0 < singles < B:
            # single decoded tokens beside portions of prompts (the runner put the single tokens' requests first)
            run(0, singles, 0, singles, 1, True)
            run(singles, B - singles, 0, T, step.max_seqlen_q, False)  # their cu_seqlens count from the step's first token
        else:
            run(0, B, 0, T, step.max_seqlen_q, False)
