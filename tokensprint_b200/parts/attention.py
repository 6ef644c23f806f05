"""Grouped-query attention over the paged cache, as a mixer part."""

from __future__ import annotations

from typing import Mapping, Optional, Sequence

import torch

from tokensprint_b200 import ops
from tokensprint_b200.parts.base import (
    BuildContext,
    CacheNeed,
    LayerCache,
    Mixer,
    PartSpec,
    ResidualNorm,
    StepContext,
    TensorSpec,
    build_part,
    register_part,
)
from tokensprint_b200.parts.linear import folding_possible, linear, linear_into_residual, linear_scaled


@register_part("mixer", "attention")
class AttentionMixer(Mixer):
    """q/k/v projections, optional per-head q/k RMSNorm, position encoding, store of keys
    and values into the cache, causal softmax attention over the cache, output projection
    (engine/nn/attention.py:164-200).

    Parameters: `hidden_size`, `num_heads`, `num_kv_heads`, `head_dim` (free of the width:
    num_heads * head_dim need not equal hidden_size), `qk_norm` + `qk_norm_eps`, `window`
    (0: every earlier key; n: the last n keys, the query's own included), `scale`
    (default head_dim^-0.5, engine/nn/sdpa.py:56), `position` (a position-encoding spec or
    None) and the checkpoint names of the tensors.  q, k, v weights are stacked at load
    into one [(nq + 2 nkv) d, H] matrix.

    Further options, each free of the others:
    `qk_norm` = "joint": one RMS norm over a token's whole q projection and one over its whole k
    projection, before they are cut into heads (weights of nq*d and nkv*d entries), instead of a
    norm per head (True or "head").
    `values` = "keys": there is no value projection; a token's values are its key projection as it
    comes, before norm and rotation (`v` is then no tensor name).
    `chunk` = n: a query sees only the keys of its own block of n positions (blocks count from
    position 0 of the sequence); the cache gives the pages of earlier blocks back.
    `sink` = s: every softmax's denominator also holds exp(s), a key without a value.
    `sinks` = name of a [num_heads] tensor: the same with a learned score per query head.
    `softcap` = c > 0: the scaled score passes through c * tanh(s / c) before the softmax.
    `q_bias`, `k_bias`, `v_bias`: names of the projections' biases.
    `qk_norm` = "unit_after_rotation": q and k heads are divided by sqrt(mean(x^2) + qk_norm_eps)
    after the rotation, without a weight.
    `value_dim`: values (and the heads the output projection reads) of another width than keys.
    `gate` = name of a [num_heads * value_dim, hidden] matrix: the concatenated heads are multiplied
    by sigmoid(gate x) before the output projection.
    `q_temperature` = (coef, every): the queries at position p are multiplied by
    1 + coef * ln(floor((p + 1) / every) + 1).
    `distance` = (name r1, name r2) of two [num_heads] tensors: the scaled score of key j for the query
    at position i loses r1_h * ln(1 + r2_h * (i - j)), a penalty per head that grows with the logarithm
    of the distance (positions enter such a layer through it, and through the temperature, alone).
    A position encoding whose cosines and sines carry a magnitude is applied from its table.
    With any of the options from `sinks` on, one product gives [q | k | v | gate], `qkv_prepare`
    adds biases, rotates, norms and stores (keys and values padded with zeros to one common width
    that the attention kernels take), and the gate is a kernel behind attention.
    """

    folds_norms = True
    # its own kernels only; a position encoding that rewrites q and k itself gets them from a kernel
    # that has run (not from a product that may still wait in a chain)
    reads_through_ops = True

    def __init__(
        self,
        ctx: BuildContext,
        *,
        hidden_size: int,
        num_heads: int,
        num_kv_heads: int,
        head_dim: int,
        q: str,
        k: str,
        o: str,
        v: Optional[str] = None,
        qk_norm: "bool | str" = False,
        qk_norm_eps: float = 1e-6,
        q_norm: Optional[str] = None,
        k_norm: Optional[str] = None,
        window: int = 0,
        scale: Optional[float] = None,
        position: Optional[PartSpec] = None,
        values: str = "projection",
        chunk: int = 0,
        sink: Optional[float] = None,
        sinks: Optional[str] = None,
        softcap: float = 0.0,
        q_bias: Optional[str] = None,
        k_bias: Optional[str] = None,
        v_bias: Optional[str] = None,
        value_dim: Optional[int] = None,
        gate: Optional[str] = None,
        q_temperature: Optional[Sequence[float]] = None,
        distance: Optional[Sequence[str]] = None,
    ) -> None:
        if qk_norm is True:
            qk_norm = "head"
        if qk_norm not in (False, "head", "joint", "unit_after_rotation"):
            raise ValueError(f"attention: qk_norm must be False, 'head', 'joint' or 'unit_after_rotation', got {qk_norm!r}")
        unit_after = qk_norm == "unit_after_rotation"
        if unit_after:
            qk_norm = False
        if sink is not None and sinks is not None:
            raise ValueError("attention: one sink score for all heads, or a tensor of scores, not both")
        if softcap < 0:
            raise ValueError("attention: softcap must not be negative")
        if q_temperature is not None and (len(q_temperature) != 2 or int(q_temperature[1]) < 1):
            raise ValueError("attention: q_temperature is (coef, every) with every >= 1")
        if distance is not None and len(distance) != 2:
            raise ValueError("attention: distance names two tensors (r1, r2)")
        if values not in ("projection", "keys"):
            raise ValueError(f"attention: values must be 'projection' or 'keys', got {values!r}")
        if (values == "projection") != (v is not None):
            raise ValueError("attention: a value projection needs its tensor's name, and values = 'keys' has none")
        if (qk_norm == "joint") != (values == "keys"):
            # the two come as one kernel (the whole-row norm with the unnormed keys as values)
            raise ValueError("attention: qk_norm = 'joint' and values = 'keys' are offered together only")
        if num_heads % num_kv_heads:
            raise ValueError(f"attention: {num_heads} heads are no multiple of {num_kv_heads} key/value heads")
        if qk_norm and (q_norm is None or k_norm is None):
            raise ValueError("attention: qk_norm needs the names of both norm weights")
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.num_kv_heads, self.head_dim = int(num_kv_heads), int(head_dim)
        self.qk_norm, self.qk_norm_eps = bool(qk_norm), float(qk_norm_eps)
        self.joint_norm, self.values_are_keys = qk_norm == "joint", values == "keys"
        self.window, self.chunk = int(window or 0), int(chunk or 0)
        self.sink = None if sink is None else float(sink)
        if self.chunk < 0:
            raise ValueError("attention: chunk must not be negative")
        self.scale = float(scale) if scale is not None else float(head_dim) ** -0.5
        self.names = {"q": q, "k": k, "v": v, "o": o, "q_norm": q_norm, "k_norm": k_norm, "sinks": sinks, "q_bias": q_bias,
                      "k_bias": k_bias, "v_bias": v_bias, "gate": gate,
                      "r1": None if distance is None else distance[0], "r2": None if distance is None else distance[1]}
        self.q_temperature = None if q_temperature is None else (float(q_temperature[0]), int(q_temperature[1]))
        self.distance: Optional[tuple[torch.Tensor, torch.Tensor]] = None
        self.position = build_part("position_encoding", position, ctx) if position is not None else None
        self.unit_after_rotation, self.softcap = unit_after, float(softcap)
        self.value_dim = self.head_dim if value_dim is None else int(value_dim)
        magnitude = getattr(self.position, "magnitude", 1.0) if self.position is not None else 1.0
        # the path through qkv_prepare (see the class's text)
        self.general = bool(unit_after or sinks or softcap or q_bias or k_bias or v_bias or gate or self.value_dim != self.head_dim
                            or magnitude != 1.0 or q_temperature is not None or distance is not None)
        # the width the attention kernels run at: the wider of keys and values, and in bfloat16 the next
        # multiple of 16 (what the tensor-core kernels take): entries beyond a head's own are zeros
        self.kernel_dim = self.head_dim
        if self.general:
            if self.joint_norm or self.qk_norm or self.values_are_keys:
                raise ValueError("attention: biases, a unit norm after the rotation, a gate, learned sinks, a score cap and values of "
                                 "another width come without the weighted q/k norms and with a value projection")
            if self.position is not None and not hasattr(self.position, "rotary_table"):
                raise ValueError("attention: these options take a rotation that offers its table of cosines and sines (or none)")
            self.kernel_dim = max(self.head_dim, self.value_dim)
            if ctx.dtype == torch.bfloat16:
                self.kernel_dim = -(-self.kernel_dim // 16) * 16
            if self.kernel_dim > ops.QKV_PREPARE_MAX_DIM:
                raise ValueError(f"attention: heads of at most {ops.QKV_PREPARE_MAX_DIM} entries, got {self.kernel_dim}")
        # the kernels of this mixer read everything a step needs from device memory; a position
        # encoding that rewrites q and k itself decides for itself
        self.graph_safe = self.position is None or self.position.graph_safe
        if self.joint_norm or self.general:
            self.folds_norms = False  # its q/k kernel is a step of its own
            if self.joint_norm and self.position is not None and self.position.rotary_inv_freq() is None:
                raise ValueError("attention: the joint q/k norm takes a rotate-half rotation (or none)")
        self.dtype = ctx.dtype
        self.qkv_weight: Optional[torch.Tensor] = None
        self.o_weight: Optional[torch.Tensor] = None
        self.q_norm_weight: Optional[torch.Tensor] = None
        self.k_norm_weight: Optional[torch.Tensor] = None
        self.head_sinks: Optional[torch.Tensor] = None
        self.biases: dict[str, Optional[torch.Tensor]] = {"q": None, "k": None, "v": None}

    def first_weight(self) -> Optional[torch.Tensor]:
        return self.qkv_weight

    def cache_need(self) -> CacheNeed:
        if self.window > 0:  # (a layer with both bounds keeps what its window needs)
            return CacheNeed(kind="window", window=self.window, kv_heads=self.num_kv_heads, head_dim=self.kernel_dim)
        if self.chunk > 0:
            return CacheNeed(kind="chunk", window=self.chunk, kv_heads=self.num_kv_heads, head_dim=self.kernel_dim)
        return CacheNeed(kind="full", kv_heads=self.num_kv_heads, head_dim=self.kernel_dim)

    def tensor_specs(self) -> list[TensorSpec]:
        H, nq, nkv, d, e = self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim
        n = self.names
        specs = [
            TensorSpec(self.names["q"], (nq * d, H)),
            TensorSpec(self.names["k"], (nkv * d, H)),
            TensorSpec(self.names["o"], (H, nq * e)),
        ]
        if not self.values_are_keys:
            specs.insert(2, TensorSpec(self.names["v"], (nkv * e, H)))
        if n["gate"] is not None:
            specs.append(TensorSpec(n["gate"], (nq * e, H)))
        if n["sinks"] is not None:
            specs.append(TensorSpec(n["sinks"], (nq,), "vector"))
        if n["r1"] is not None:
            specs += [TensorSpec(n["r1"], (nq,), "vector"), TensorSpec(n["r2"], (nq,), "vector")]
        for key, width in (("q_bias", nq * d), ("k_bias", nkv * d), ("v_bias", nkv * e)):
            if n[key] is not None:
                specs.append(TensorSpec(n[key], (width,), "vector"))
        if self.qk_norm:
            specs.append(TensorSpec(self.names["q_norm"], (nq * d if self.joint_norm else d,), "vector"))
            specs.append(TensorSpec(self.names["k_norm"], (nkv * d if self.joint_norm else d,), "vector"))
        if self.position is not None:
            specs.extend(self.position.tensor_specs())
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        stacked = [tensors[n["q"]], tensors[n["k"]]] + ([] if self.values_are_keys else [tensors[n["v"]]])
        if n["gate"] is not None:
            stacked.append(tensors[n["gate"]])
        self.qkv_weight = torch.cat(stacked, dim=0).contiguous()
        if n["sinks"] is not None:
            self.head_sinks = tensors[n["sinks"]]
        if n["r1"] is not None:
            self.distance = (tensors[n["r1"]], tensors[n["r2"]])
        for key in ("q", "k", "v"):
            if n[key + "_bias"] is not None:
                self.biases[key] = tensors[n[key + "_bias"]]
        self.o_weight = tensors[n["o"]]
        if self.qk_norm:
            self.q_norm_weight = tensors[n["q_norm"]]
            self.k_norm_weight = tensors[n["k_norm"]]
        if self.position is not None:
            self.position.load(tensors)

    def can_fold(self, num_tokens: int, dtype: torch.dtype) -> bool:
        return folding_possible(num_tokens, dtype, self.qkv_weight, self.o_weight)

    def forward(self, x, step: StepContext, cache: LayerCache, fold: Optional[ResidualNorm] = None):
        """x: [T, H], or a PreNormed (its missing 1/rms is applied by the q/k/v product).  With
        `fold` the output projection adds its result into fold.hidden itself and the PreNormed of
        the norm that follows is returned instead of the branch output."""
        if cache.k_pages is None or cache.group < 0:
            raise ops.KernelError("attention: this mixer needs cache pages (none were bound to its run)")
        xt = x if isinstance(x, torch.Tensor) else x.x
        T = xt.shape[0]
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        tables = step.groups[cache.group]
        q = torch.empty((T, nq * d), device=xt.device, dtype=xt.dtype)
        if self.joint_norm:
            return self._forward_joint(x, q, step, cache, tables)
        if self.general:
            return self._forward_general(x, step, cache, tables)
        inv_freq = self.position.rotary_inv_freq() if self.position is not None else None
        fused = self.position is None or inv_freq is not None
        if (fused and cache.writes and d == ops.GEMM_QK_ROPE_HEAD_DIM and (inv_freq is None or inv_freq.numel() == d // 2)
                and folding_possible(T, xt.dtype, self.qkv_weight)):
            # few tokens, heads of 128: norm, rotation and the store are the projection's own epilogue
            pre = None if isinstance(x, torch.Tensor) else x
            ops.gemm_qk_rope_store(
                xt, self.qkv_weight, q, cache.k_pages, cache.v_pages, tables.slot_mapping, step.positions,
                self.q_norm_weight, self.k_norm_weight, self.qk_norm_eps, inv_freq, nq, nkv,
                scale_ssq=None if pre is None else pre.ssq, scale_width=1 if pre is None else pre.width,
                scale_eps=0.0 if pre is None else pre.eps, prefetch=self.o_weight,
                cos_sin=None if inv_freq is None else self.position.rotary_cos_sin(step))
            out = torch.empty((T, nq * d), device=xt.device, dtype=xt.dtype)
            self._attend(q, out, step, cache, tables)
            if fold is not None:
                return linear_into_residual(out, self.o_weight, fold, next_weight=step.weight_after)
            return linear(out, self.o_weight, next_weight=step.weight_after)
        qkv = linear_scaled(x, self.qkv_weight, next_weight=self.o_weight)
        if fused and cache.writes:
            ops.qk_norm_rope_store(
                qkv, q, cache.k_pages, cache.v_pages, tables.slot_mapping, step.positions,
                self.q_norm_weight, self.k_norm_weight, self.qk_norm_eps, inv_freq, nq, nkv, d)
        elif fused:
            # Reads a cache that another run filled: only the queries are prepared.
            self._queries_only(qkv, q, step, inv_freq)
        else:
            self._unfused(qkv, q, step, cache, tables)
        out = torch.empty((T, nq * d), device=xt.device, dtype=xt.dtype)
        self._attend(q, out, step, cache, tables)
        if fold is not None:
            return linear_into_residual(out, self.o_weight, fold, next_weight=step.weight_after)
        return linear(out, self.o_weight, next_weight=step.weight_after)

    def _forward_joint(self, x, q, step: StepContext, cache: LayerCache, tables):
        """The whole-row q/k norm with the key projection as values: one product for [q | k], one
        kernel for both norms, the rotation and the stores, attention, the output product."""
        T = q.shape[0]
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        qk = linear_scaled(x, self.qkv_weight, next_weight=self.o_weight)
        cos_sin = self.position.rotary_cos_sin(step) if self.position is not None else None
        if cache.writes:
            ops.qk_joint_norm_rope_store(qk, q, cache.k_pages, cache.v_pages, tables.slot_mapping, self.q_norm_weight,
                                         self.k_norm_weight, self.qk_norm_eps, cos_sin, nq, nkv, d)
        else:  # reads a cache that another run filled: only the queries are kept
            k_tmp = torch.empty((T, nkv, d), device=q.device, dtype=q.dtype)
            ops.qk_joint_norm_rope_store(qk, q, k_tmp, torch.empty_like(k_tmp), None, self.q_norm_weight, self.k_norm_weight,
                                         self.qk_norm_eps, cos_sin, nq, nkv, d)
        out = torch.empty((T, nq * d), device=q.device, dtype=q.dtype)
        self._attend(q, out, step, cache, tables)
        return linear(out, self.o_weight, next_weight=step.weight_after)

    def _forward_general(self, x, step: StepContext, cache: LayerCache, tables):
        """One product for [q | k | v | gate]; biases, rotation from the table, the unit norm and the
        stores in one kernel (keys and values padded to the kernels' width); attention; the gate
        (and the cut back to the values' own width); the output product."""
        T = x.shape[0]
        nq, nkv, d, e, D = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim, self.kernel_dim
        proj = linear(x, self.qkv_weight, next_weight=self.o_weight)
        table = self.position.rotary_table(step) if self.position is not None else None
        q = torch.empty((T, nq * D), device=x.device, dtype=x.dtype)
        k_off, v_off, g_off = nq * d, nq * d + nkv * d, nq * d + nkv * d + nkv * e
        writes = cache.writes
        ops.qkv_prepare(proj, 0, k_off, v_off, self.biases["q"], self.biases["k"], self.biases["v"], table, self.unit_after_rotation,
                        self.qk_norm_eps, q, cache.k_pages if writes else None, cache.v_pages if writes else None,
                        tables.slot_mapping if writes else None, nq, nkv, d, e, D, positions=step.positions,
                        query_temperature=self.q_temperature)
        out = torch.empty((T, nq * D), device=x.device, dtype=x.dtype)
        self._attend(q, out, step, cache, tables)
        gated = self.names["gate"] is not None
        if gated or D != e:
            y = torch.empty((T, nq * e), device=x.device, dtype=x.dtype)
            ops.gate_rows(out, proj[:, g_off:g_off + nq * e] if gated else None, y, nq, e, D)
            out = y
        return linear(out, self.o_weight, next_weight=step.weight_after)

    # -- attention proper ---------------------------------------------------

    def _attend(self, q, out, step: StepContext, cache: LayerCache, tables) -> None:
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.kernel_dim
        scored = {"softcap": self.softcap, "head_sinks": self.head_sinks}
        if self.distance is not None:
            scored["distance"] = self.distance
        if q.dtype == torch.bfloat16 and ops.attention_mma_supported(d) and (self.distance is None or ops.ATTENTION_MMA_DISTANCE):
            B, singles = step.num_seqs, step.decode_seqs
            few_rows = (nq // nkv) <= ops.attention_decode_rows(d)
            if step.max_seqlen_q * (nq // nkv) <= ops.attention_decode_rows(d):
                # few rows per sequence: the decode kernels, keys spread over CTAs
                self._attend_decode(q, out, step, cache, tables, 0, B, step.max_seqlen_q)
                return
            prompts_on_tcgen05 = ops.attention_tcgen05_supported(nq, nkv, d, step.page_size)
            if prompts_on_tcgen05 and few_rows and 0 < singles < B:
                # Single decoded tokens beside portions of prompts (the runner put the single tokens'
                # requests first): each kind to its own kernel.  Through the prompt kernel a decoded
                # token is a CTA that walks its whole context for a tile of a few rows (measured at
                # Qwen3-14B's heads, 140 decoded tokens at context 1,500 beside 8 prompts of 1,000:
                # 587 us in one launch, 179 + 218 us in two).
                self._attend_decode(q[:singles], out[:singles], step, cache, tables, 0, singles, 1)
                ops.attention_prefill_tcgen05(
                    q, cache.k_pages, cache.v_pages, out, step.cu_seqlens_q[singles:], step.context_lens[singles:],
                    tables.block_table[singles:], step.page_size, B - singles, step.max_seqlen_q, nq, nkv, self.scale, self.window,
                    chunk=self.chunk, sink=self.sink, **scored)
                return
            if prompts_on_tcgen05:
                # prompt portions: the tcgen05 kernel, where it takes the sizes
                ops.attention_prefill_tcgen05(
                    q, cache.k_pages, cache.v_pages, out, step.cu_seqlens_q, step.context_lens, tables.block_table,
                    step.page_size, step.num_seqs, step.max_seqlen_q, nq, nkv, self.scale, self.window, chunk=self.chunk, sink=self.sink,
                    **scored)
                return
            ops.attention_paged_mma(
                q, cache.k_pages, cache.v_pages, out, step.cu_seqlens_q, step.context_lens, tables.block_table,
                step.seq_index, step.page_size, step.num_seqs, step.max_seqlen_q, nq, nkv, d, self.scale,
                self.window, 1, None, 0, chunk=self.chunk, sink=self.sink, **scored)
            return
        # float32 runs, and head sizes the tensor-core kernel does not take
        ops.attention_paged_simple(
            q, cache.k_pages, cache.v_pages, out, step.positions, step.seq_index, tables.block_table,
            step.page_size, self.num_heads, self.num_kv_heads, d, self.scale, self.window, self.chunk, self.sink,
            softcap=self.softcap, head_sinks=self.head_sinks, distance=self.distance)

    def _attend_decode(self, q, out, step: StepContext, cache: LayerCache, tables, first: int, count: int, max_q: int) -> None:
        """Sequences [first, first + count) of the batch, each with at most `max_q` tokens (few enough
        rows for the decode kernels); q and out hold exactly their tokens."""
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.kernel_dim
        cu = step.cu_seqlens_q[first : first + count + 1]
        lens = step.context_lens[first : first + count]
        table = tables.block_table[first : first + count]
        seq_index = step.seq_index[: q.shape[0]] if first == 0 else step.seq_index
        # The count must not depend on the step's actual lengths (a captured graph is
        # replayed for all of them): plan for a typical context, each sequence then
        # divides its own keys evenly.
        reach = min(self.window, self.chunk) if self.window and self.chunk else self.window or self.chunk  # the most keys a query sees
        context = ops.attention_decode_plan_context(step.max_context_len, reach)
        splits = ops.attention_decode_splits(count, nkv, context, d)
        # (the even-share decode kernel knows neither a block bound nor a sink nor a score cap)
        if (self.chunk == 0 and self.sink is None and self.head_sinks is None and self.softcap == 0.0 and self.distance is None
                and ops.attention_decode_prefers_flat(count, nkv, splits, d)
                and ops.attention_decode_flat_supported(nq, nkv, d, step.page_size, count, max_q)):
            # more (sequence, KV head) pairs than CTAs run at once: an even share of all key blocks per CTA
            ops.attention_decode_flat(
                q, cache.k_pages, cache.v_pages, out, cu, lens, table, seq_index, step.page_size, count, max_q, nq, nkv, d,
                self.scale, self.window)
            return
        scratch = None
        if splits > 1:
            scratch = torch.empty(ops.attention_scratch_floats(q.shape[0] * nq, splits, d), device=q.device, dtype=torch.float32)
        ops.attention_paged_mma(
            q, cache.k_pages, cache.v_pages, out, cu, lens, table, seq_index, step.page_size, count, max_q, nq, nkv, d,
            self.scale, self.window, splits, scratch, 0, chunk=self.chunk, sink=self.sink, softcap=self.softcap, head_sinks=self.head_sinks,
            distance=self.distance)

    # -- less common paths ----------------------------------------------------

    def _queries_only(self, qkv, q, step: StepContext, inv_freq) -> None:
        T = qkv.shape[0]
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        k_tmp = torch.empty((T, nkv, d), device=qkv.device, dtype=qkv.dtype)
        v_tmp = torch.empty((T, nkv, d), device=qkv.device, dtype=qkv.dtype)
        ops.qk_norm_rope_store(
            qkv, q, k_tmp, v_tmp, None, step.positions, self.q_norm_weight, self.k_norm_weight,
            self.qk_norm_eps, inv_freq, nq, nkv, d)

    def _unfused(self, qkv, q, step: StepContext, cache: LayerCache, tables) -> None:
        """A position encoding that the fused kernel does not know: norm into dense
        buffers, let the part rewrite q and k, then store keys and values."""
        T = qkv.shape[0]
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        k_tmp = torch.empty((T, nkv, d), device=qkv.device, dtype=qkv.dtype)
        v_tmp = torch.empty((T, nkv, d), device=qkv.device, dtype=qkv.dtype)
        ops.qk_norm_rope_store(
            qkv, q, k_tmp, v_tmp, None, step.positions, self.q_norm_weight, self.k_norm_weight,
            self.qk_norm_eps, None, nq, nkv, d)
        self.position.apply(q.view(T, nq, d), k_tmp, step)
        if cache.writes:
            kv = torch.cat([k_tmp.view(T, nkv * d), v_tmp.view(T, nkv * d)], dim=1).contiguous()
            scratch_q = torch.empty((T, 0), device=qkv.device, dtype=qkv.dtype)
            ops.qk_norm_rope_store(
                kv, scratch_q, cache.k_pages, cache.v_pages, tables.slot_mapping, step.positions,
                None, None, self.qk_norm_eps, None, 0, nkv, d)
