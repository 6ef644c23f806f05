"""Python face of the CUDA kernels: argument checks, then one call into the library.

Every function works on CUDA tensors, launches on torch's current stream and returns
without synchronising.  A size that a kernel does not take raises `KernelError` with
the limit in words; nothing falls back to another implementation.
"""

from __future__ import annotations

import ctypes
import os as _os
from typing import Optional

import torch

from tokensprint_b200.csrc import build as _build

DTYPE_CODES = {torch.float32: 0, torch.bfloat16: 1}
_GEMM_MAX_TILES = 1 << 16  # size of the ticket-counter arrays of the GEMM and of the decode attention

_c_void_p = ctypes.c_void_p
_c_int = ctypes.c_int
_c_float = ctypes.c_float
_c_ll = ctypes.c_longlong

_SIGNATURES = {
    "ts_embed_gather": [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_float, _c_void_p],
    "ts_feed_tokens": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p],
    "ts_add_rmsnorm": [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_float, _c_void_p],
    "ts_residual_add": [_c_void_p, _c_void_p, _c_int, _c_ll, _c_void_p],
    "ts_swiglu": [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "ts_qk_norm_rope_store": [
        _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
        _c_float, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p,
    ],
    "ts_attention_paged_simple": [
        _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
        _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int, _c_float, _c_float, _c_void_p, _c_void_p, _c_void_p,
        _c_void_p,
    ],
    "ts_sample": [_c_void_p, _c_int, _c_ll, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p],
    "ts_sgemm_nt": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_ll, _c_ll, _c_ll, _c_void_p],
    "ts_sgemm_nt_batched": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_ll, _c_ll, _c_ll, _c_int, _c_ll, _c_ll, _c_ll, _c_void_p],
    "ts_pair_hash_embed": [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int,
                           _c_int, _c_ll, _c_ll, _c_ll, _c_void_p],
    "ts_rmsnorm_add": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_float, _c_void_p],
    "ts_round_rows": [_c_void_p, _c_int, _c_void_p, _c_int, _c_ll, _c_void_p],
    "ts_latent_prepare": [_c_void_p, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_float,
                          _c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_void_p, _c_ll, _c_void_p],
    "ts_latent_attention_simple": [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int,
                                   _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_void_p],
    "ts_gelu_tanh": [_c_void_p, _c_void_p, _c_int, _c_ll, _c_void_p],
    "ts_capped_glu": [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_float, _c_float, _c_void_p],
    "ts_gelu_gate_rows": [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_ll, _c_int, _c_int, _c_void_p],
    "ts_router_topk": [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "ts_router": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p,
                  _c_void_p],
    "ts_moe_gate_up_mma": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int,
                           _c_int, _c_int, _c_float, _c_float, _c_int, _c_int, _c_void_p],
    "ts_moe_down_mma": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "ts_moe_plan": [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "ts_moe_gate_up": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int,
                       _c_int, _c_int, _c_float, _c_float, _c_int, _c_void_p],
    "ts_moe_down": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "ts_qk_joint_norm_rope_store": [_c_void_p, _c_int, _c_ll, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_float,
                                    _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "ts_gla_decay": [_c_void_p, _c_ll, _c_int, _c_void_p, _c_float, _c_void_p, _c_int, _c_int, _c_void_p],
    "ts_gla_scan": [_c_void_p, _c_void_p, _c_void_p, _c_ll, _c_int, _c_void_p, _c_float, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                    _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "ts_gla_norm_gate": [_c_void_p, _c_void_p, _c_ll, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_float, _c_void_p],
    "ts_branch_norm_add": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_float, _c_float,
                           _c_void_p],
    "ts_stream_add": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p],
    "ts_moe_combine": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p],
}

_functions: dict[str, object] = {}


class KernelError(RuntimeError):
    pass


def library() -> ctypes.CDLL:
    return _build.load()


def _fn(name: str):
    f = _functions.get(name)
    if f is None:
        lib = library()
        try:
            f = getattr(lib, name)
        except AttributeError as e:
            raise KernelError(f"the CUDA library has no entry point {name}") from e
        f.argtypes = _SIGNATURES[name]
        f.restype = _c_int
        _functions[name] = f
    return f


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """The current CUDA stream's handle.  (torch.cuda.current_stream() builds a Python object and
    resolves the device by name every time: a third of the host's time in a step launched kernel by
    kernel; the raw call is a hundred times cheaper.)"""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


# Launches of this library's kernels since import (library GEMMs are not counted).
launch_count = 0


def _check(name: str, status: int) -> None:
    global launch_count
    if status == 0:
        launch_count += 1
        return
    if status == -1:
        raise KernelError(f"{name}: bad argument")
    if status == -2:
        raise KernelError(f"{name}: size not supported by this kernel")
    raise KernelError(f"{name}: CUDA error {status} at launch")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _cuda_contig(name: str, t: torch.Tensor, dtype: Optional[torch.dtype] = None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous, got strides {t.stride()} for shape {tuple(t.shape)}")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")


def _act_code(name: str, t: torch.Tensor) -> int:
    code = DTYPE_CODES.get(t.dtype)
    if code is None:
        raise KernelError(f"{name} must be float32 or bfloat16, got {t.dtype}")
    return code


# ---------------------------------------------------------------------------
# chains of products: several skinny GEMMs that feed one another, launched as one kernel

# Whether a model step chains its products by itself (Model.chain_scope).  Off: measured on B200 at
# Qwen3-8B sizes, the four products of a decode layer take 87 us as four launches (programmatic
# dependent launch already overlaps a kernel's start with its predecessor's end) and 102 to 109 us
# as one chained launch: what separates two products is the chain of trips to the L2 at the end of
# the first (partial sums, ticket, sums, the finished tile) and the first copies of the second, about
# 8 us either way, and inside one kernel the copies that early CTAs ask for the next phase delay the
# last copies of the late ones.  TS_GEMM_CHAIN=1 switches it on for measurements.
GEMM_CHAIN = _os.environ.get("TS_GEMM_CHAIN", "0") == "1"
_chain_open = False
_chain_keep: list = []  # tensors that products waiting in the chain read or write
_chain_counted = 0


def _chain_sync_words(device: torch.device) -> torch.Tensor:
    """Per (device, stream): the counters of the chained kernel's grid barrier (zero between launches)."""
    counters, _ = _gemm_workspace(device)
    return counters[_GEMM_MAX_TILES:]


class gemm_chain:
    """While this context is open, the engine's own few-row products are not launched when they are
    called: they are collected, and up to `ts_gemm_chain_max_phases` of them that follow one another
    are launched as ONE kernel, in which each starts fetching its weights while the one before it is
    still being finished.  Every other op of this module launches what is pending before it runs, so
    a caller that only uses these ops sees no difference; code that reads a product's output by
    other means (a torch op) calls `flush_gemm_chain()` first.  Nothing happens when `enabled` is
    false, and chains do not nest."""

    def __init__(self, device: torch.device, enabled: bool = True) -> None:
        self.device, self.enabled = device, bool(enabled)

    def __enter__(self):
        global _chain_open, _chain_counted
        self.mine = self.enabled and not _chain_open
        if self.mine:
            fn = library().ts_gemm_chain_begin
            fn.argtypes = [_c_void_p]
            fn.restype = None
            fn(_chain_sync_words(self.device).data_ptr())
            _chain_open = True
            _chain_counted = 0
        return self

    def __exit__(self, *exc):
        global _chain_open
        if self.mine:
            try:
                flush_gemm_chain(end=True)
            finally:
                _chain_open = False
                _chain_keep.clear()
        return False


def flush_gemm_chain(end: bool = False) -> None:
    """Launches the products that wait in the chain (nothing, if no chain is open)."""
    global launch_count, _chain_counted
    if not _chain_open:
        return
    lib = library()
    status = (lib.ts_gemm_chain_end if end else lib.ts_gemm_chain_flush)()
    launched = lib.ts_gemm_chain_launches()
    launch_count += launched - _chain_counted
    _chain_counted = launched
    _chain_keep.clear()
    if status != 0:
        raise KernelError(f"chained products: CUDA error {status} at launch")


def _check_product(name: str, status: int, *tensors) -> None:
    """_check for a product that may have joined a chain instead of being launched."""
    global launch_count, _chain_counted
    if not _chain_open:
        _check(name, status)
        return
    _chain_keep.append(tensors)
    launched = library().ts_gemm_chain_launches()  # a full list, or another row count, launched what was pending
    launch_count += launched - _chain_counted
    _chain_counted = launched
    if status != 0:
        _check(name, status)


def embed_gather(hidden: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, scale: float = 1.0) -> None:
    """hidden[t] = table[ids[t]] * scale, widened to float32.  hidden [T,H] f32, table [V,H], ids [T] i32."""
    flush_gemm_chain()
    _cuda_contig("hidden", hidden, torch.float32)
    _cuda_contig("table", table)
    _cuda_contig("ids", ids, torch.int32)
    T, H = hidden.shape
    V = table.shape[0]
    if table.shape[1] != H or ids.numel() < T:
        raise KernelError(f"embed_gather: shapes disagree: hidden {tuple(hidden.shape)}, table {tuple(table.shape)}, ids {tuple(ids.shape)}")
    _check("embed_gather", _fn("ts_embed_gather")(
        hidden.data_ptr(), table.data_ptr(), _act_code("table", table), ids.data_ptr(), T, H, V, float(scale), _stream()))


def feed_tokens(ids: torch.Tensor, source: torch.Tensor, lanes: torch.Tensor, rows: torch.Tensor, n: int) -> None:
    """ids[lanes[i]] = source[rows[i]] for i < n (all int32, on the device): token ids that an
    earlier kernel produced go into a step's inputs without passing through the host."""
    flush_gemm_chain()
    for name, t in (("ids", ids), ("source", source), ("lanes", lanes), ("rows", rows)):
        _cuda_contig(name, t, torch.int32)
    if n > lanes.numel() or n > rows.numel():
        raise KernelError(f"feed_tokens: {n} lanes, but the index arrays hold {lanes.numel()} and {rows.numel()}")
    _check("feed_tokens", _fn("ts_feed_tokens")(ids.data_ptr(), source.data_ptr(), lanes.data_ptr(), rows.data_ptr(), int(n), _stream()))


def add_rmsnorm(
    hidden: torch.Tensor,
    delta: Optional[torch.Tensor],
    weight: torch.Tensor,
    out: torch.Tensor,
    eps: float,
    row_index: Optional[torch.Tensor] = None,
) -> None:
    """hidden += delta (float32, in place) and out = RMSNorm(hidden) * weight.

    hidden [T,H] f32; delta [T,H] of out's dtype or None; weight [H] f32; out [rows,H].
    With `row_index` ([rows] i32) only those rows are normed and hidden is left as it is.
    """
    flush_gemm_chain()
    _cuda_contig("hidden", hidden, torch.float32)
    _cuda_contig("weight", weight, torch.float32)
    _cuda_contig("out", out)
    H = hidden.shape[-1]
    rows = out.shape[0]
    if out.shape[-1] != H or weight.numel() != H:
        raise KernelError(f"add_rmsnorm: widths disagree: hidden {tuple(hidden.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if delta is not None:
        _cuda_contig("delta", delta, out.dtype)
        if delta.shape != hidden.shape:
            raise KernelError("add_rmsnorm: delta must have hidden's shape")
    if row_index is not None:
        _cuda_contig("row_index", row_index, torch.int32)
        if row_index.numel() < rows:
            raise KernelError("add_rmsnorm: row_index is shorter than out")
    elif rows != hidden.shape[0]:
        raise KernelError("add_rmsnorm: out must have hidden's rows when no row_index is given")
    _check("add_rmsnorm", _fn("ts_add_rmsnorm")(
        hidden.data_ptr(), _ptr(delta), _act_code("out", out), weight.data_ptr(), out.data_ptr(),
        _ptr(row_index), rows, H, float(eps), _stream()))


def residual_add(hidden: torch.Tensor, delta: torch.Tensor) -> None:
    """hidden += delta in float32.  hidden [T,H] f32, delta [T,H] f32 or bf16."""
    flush_gemm_chain()
    _cuda_contig("hidden", hidden, torch.float32)
    _cuda_contig("delta", delta)
    if delta.shape != hidden.shape:
        raise KernelError("residual_add: shapes disagree")
    _check("residual_add", _fn("ts_residual_add")(
        hidden.data_ptr(), delta.data_ptr(), _act_code("delta", delta), hidden.numel(), _stream()))


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, block: int = 0) -> None:
    """out[t,i] = silu(gate[t,i]) * up[t,i].  gate_up [T,2I], out [T,I].  block 0: gate i at column
    i, up at I + i; block 64: blocks of 128 columns, 64 gates and then their 64 ups."""
    flush_gemm_chain()
    _cuda_contig("gate_up", gate_up)
    _cuda_contig("out", out, gate_up.dtype)
    T, I = out.shape
    if gate_up.shape != (T, 2 * I):
        raise KernelError(f"swiglu: gate_up {tuple(gate_up.shape)} does not match out {tuple(out.shape)}")
    if block not in (0, 64) or (block and I % 64):
        raise KernelError(f"swiglu: block must be 0 or 64 (and then divide the width), got {block} for width {I}")
    _check("swiglu", _fn("ts_swiglu")(gate_up.data_ptr(), out.data_ptr(), _act_code("out", out), T, I, int(block), _stream()))


QK_ROPE_MAX_HEAD_DIM = 512


def qk_norm_rope_store(
    qkv: torch.Tensor,
    q_out: torch.Tensor,
    k_dst: Optional[torch.Tensor],
    v_dst: Optional[torch.Tensor],
    slot_mapping: Optional[torch.Tensor],
    positions: torch.Tensor,
    q_norm_weight: Optional[torch.Tensor],
    k_norm_weight: Optional[torch.Tensor],
    eps: float,
    inv_freq: Optional[torch.Tensor],
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
) -> None:
    """Per-head q/k RMSNorm, rotary encoding, and the key/value store.

    qkv [T,(nq+2nkv)*d]; q_out [T,nq*d]; k_dst/v_dst: the cache pools [slots,nkv,d] (with
    `slot_mapping` [T] i32, -1 = skip) or dense [T,nkv,d] buffers (slot_mapping None).
    Norm weights [d] f32 or None (no norm); inv_freq [rot/2] f32 or None (no rotation);
    a rotation narrower than d leaves the upper dims as they are.
    """
    flush_gemm_chain()
    _cuda_contig("qkv", qkv)
    _cuda_contig("q_out", q_out, qkv.dtype)
    _cuda_contig("positions", positions, torch.int32)
    T = qkv.shape[0]
    nq, nkv, d = num_heads, num_kv_heads, head_dim
    if d > QK_ROPE_MAX_HEAD_DIM or d % 2:
        raise KernelError(f"qk_norm_rope_store: head_dim must be even and <= {QK_ROPE_MAX_HEAD_DIM}, got {d}")
    if qkv.shape[1] != (nq + 2 * nkv) * d or q_out.numel() != T * nq * d:
        raise KernelError(f"qk_norm_rope_store: qkv {tuple(qkv.shape)} / q_out {tuple(q_out.shape)} do not match heads {nq}+2*{nkv} of {d}")
    if nkv > 0:
        for name, c in (("k_dst", k_dst), ("v_dst", v_dst)):
            if c is None:
                raise KernelError(f"qk_norm_rope_store: {name} is required")
            _cuda_contig(name, c, qkv.dtype)
            if c.shape[-1] != d or c.shape[-2] != nkv:
                raise KernelError(f"qk_norm_rope_store: {name} must end in [{nkv},{d}], got {tuple(c.shape)}")
        if slot_mapping is None and (k_dst.numel() < T * nkv * d or v_dst.numel() < T * nkv * d):
            raise KernelError("qk_norm_rope_store: dense k/v buffers are too small")
    if slot_mapping is not None:
        _cuda_contig("slot_mapping", slot_mapping, torch.int32)
        if slot_mapping.numel() < T:
            raise KernelError("qk_norm_rope_store: slot_mapping is shorter than the batch")
    if positions.numel() < T:
        raise KernelError("qk_norm_rope_store: positions is shorter than the batch")
    for name, w in (("q_norm_weight", q_norm_weight), ("k_norm_weight", k_norm_weight)):
        if w is not None:
            _cuda_contig(name, w, torch.float32)
            if w.numel() != d:
                raise KernelError(f"qk_norm_rope_store: {name} must have {d} entries")
    rot = 0
    if inv_freq is not None:
        _cuda_contig("inv_freq", inv_freq, torch.float32)
        rot = 2 * inv_freq.numel()
        if rot > d or rot <= 0:
            raise KernelError(f"qk_norm_rope_store: rotary width {rot} does not fit head_dim {d}")
    _check("qk_norm_rope_store", _fn("ts_qk_norm_rope_store")(
        qkv.data_ptr(), _act_code("qkv", qkv), q_out.data_ptr(), _ptr(k_dst), _ptr(v_dst),
        _ptr(slot_mapping), positions.data_ptr(), _ptr(q_norm_weight), _ptr(k_norm_weight),
        float(eps), _ptr(inv_freq), rot, T, nq, nkv, d, _stream()))


ATTENTION_SIMPLE_MAX_HEAD_DIM = 512


def attention_paged_simple(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    out: torch.Tensor,
    positions: torch.Tensor,
    seq_index: torch.Tensor,
    block_table: torch.Tensor,
    page_size: int,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    scale: float,
    window: int = 0,
    chunk: int = 0,
    sink: Optional[float] = None,
    softcap: float = 0.0,
    head_sinks: Optional[torch.Tensor] = None,
    distance: Optional[tuple[torch.Tensor, torch.Tensor]] = None,
) -> None:
    """Causal attention over the paged cache on CUDA cores (float32 or bfloat16).

    q/out [T,nq*d]; caches [pages,page,nkv,d]; positions, seq_index [T] i32;
    block_table [B,max_blocks] i32.  window > 0: a query sees its last `window` keys.
    chunk > 0: a query sees only the keys of its own block of `chunk` positions (blocks count
    from position 0).  sink: a score that joins every softmax's denominator without a value;
    head_sinks [nq] float32: one such score per query head.  softcap > 0: the scaled score goes
    through softcap * tanh(s / softcap).  distance = (r1, r2), [nq] float32 each: the score of key j
    loses r1 * ln(1 + r2 * (position - j)).
    """
    flush_gemm_chain()
    if distance is not None:
        for name, t in zip(("distance r1", "distance r2"), distance):
            _cuda_contig(name, t, torch.float32)
            if t.numel() != num_heads:
                raise KernelError(f"attention: {name} must have one entry per query head ({num_heads}), got {t.numel()}")
    if head_sinks is not None:
        _cuda_contig("head_sinks", head_sinks, torch.float32)
        if head_sinks.numel() != num_heads:
            raise KernelError(f"attention: head_sinks must have one entry per query head ({num_heads}), got {head_sinks.numel()}")
    _cuda_contig("q", q)
    _cuda_contig("k_cache", k_cache, q.dtype)
    _cuda_contig("v_cache", v_cache, q.dtype)
    _cuda_contig("out", out, q.dtype)
    _cuda_contig("positions", positions, torch.int32)
    _cuda_contig("seq_index", seq_index, torch.int32)
    _cuda_contig("block_table", block_table, torch.int32)
    T = q.shape[0]
    nq, nkv, d = num_heads, num_kv_heads, head_dim
    if d > ATTENTION_SIMPLE_MAX_HEAD_DIM:
        raise KernelError(f"attention_paged_simple: head_dim must be <= {ATTENTION_SIMPLE_MAX_HEAD_DIM}, got {d}")
    if nq % nkv:
        raise KernelError(f"attention: {nq} query heads are no multiple of {nkv} key/value heads")
    if q.numel() != T * nq * d or out.numel() != T * nq * d:
        raise KernelError("attention: q/out do not match [T, heads*head_dim]")
    if tuple(k_cache.shape[-3:]) != (page_size, nkv, d) or k_cache.shape != v_cache.shape:
        raise KernelError(f"attention: caches must be [pages,{page_size},{nkv},{d}], got {tuple(k_cache.shape)} and {tuple(v_cache.shape)}")
    if block_table.dim() != 2 or positions.numel() < T or seq_index.numel() < T:
        raise KernelError("attention: block_table must be [B,max_blocks]; positions and seq_index need T entries")
    _check("attention_paged_simple", _fn("ts_attention_paged_simple")(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), _act_code("q", q), out.data_ptr(),
        positions.data_ptr(), seq_index.data_ptr(), block_table.data_ptr(), block_table.shape[1],
        page_size, T, nq, nkv, d, float(scale), int(window), int(chunk), 0 if sink is None else 1,
        0.0 if sink is None else float(sink), float(softcap), _ptr(head_sinks),
        None if distance is None else distance[0].data_ptr(), None if distance is None else distance[1].data_ptr(), _stream()))


def sample(
    logits: torch.Tensor,
    temperature: torch.Tensor,
    keys: Optional[torch.Tensor],
    out: torch.Tensor,
) -> None:
    """One token per row of float32 logits [R,V]: argmax where temperature is 0, else the
    exponential race keyed by keys[r] (int64, the noise stream of that row).  out [R] i32."""
    flush_gemm_chain()
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be a float32 CUDA matrix with unit inner stride")
    _cuda_contig("temperature", temperature, torch.float32)
    _cuda_contig("out", out, torch.int32)
    R, V = logits.shape
    if keys is not None:
        _cuda_contig("keys", keys, torch.int64)
        if keys.numel() < R:
            raise KernelError("sample: keys is shorter than the batch")
    if temperature.numel() < R or out.numel() < R:
        raise KernelError("sample: temperature/out are shorter than the batch")
    # stage 1 leaves one (value, index) pair per 2048-entry chunk of each row for stage 2
    scratch = torch.empty(R * (-(-V // 2048)) * 2, dtype=torch.int32, device=logits.device)
    _check("sample", _fn("ts_sample")(
        logits.data_ptr(), V, logits.stride(0), temperature.data_ptr(), _ptr(keys), out.data_ptr(), R,
        scratch.data_ptr(), _stream()))
    global launch_count
    launch_count += 1  # two kernels per call


def sgemm_nt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T in true float32 (FFMA)."""
    flush_gemm_chain()
    for name, t in (("a", a), ("w", w), ("out", out)):
        if not t.is_cuda or t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"sgemm_nt: {name} must be a float32 CUDA matrix with unit inner stride")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"sgemm_nt: shapes disagree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    _check("sgemm_nt", _fn("ts_sgemm_nt")(
        a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), w.stride(0), out.stride(0), _stream()))


def sgemm_nt_batched(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[b] = a[b] @ w[b]^T in true float32 for b < batch: a [batch, M, K], w [batch, N, K], out
    [batch, M, N], each possibly a strided view (unit inner stride)."""
    flush_gemm_chain()
    for name, t in (("a", a), ("w", w), ("out", out)):
        if not t.is_cuda or t.dtype != torch.float32 or t.dim() != 3 or t.stride(2) != 1:
            raise KernelError(f"sgemm_nt_batched: {name} must be a float32 CUDA tensor [batch, rows, cols] with unit inner stride")
    batch, M, K = a.shape
    N = w.shape[1]
    if w.shape != (batch, N, K) or out.shape != (batch, M, N):
        raise KernelError(f"sgemm_nt_batched: shapes disagree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    _check("sgemm_nt_batched", _fn("ts_sgemm_nt_batched")(
        a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, a.stride(1), w.stride(1), out.stride(1), batch,
        a.stride(0), w.stride(0), out.stride(0), _stream()))


def library_bmm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[b] = a[b] @ w[b]^T by the library's batched GEMM (bfloat16, float32 sums): the many small
    per-head products of a latent attention layer.  Strided views are taken as they are."""
    flush_gemm_chain()
    torch.bmm(a, w.transpose(1, 2), out=out)


def pair_hash_embed(hidden: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, positions: torch.Tensor, seq_index: torch.Tensor,
                    cu_seqlens: torch.Tensor, state_slots: torch.Tensor, last_token: torch.Tensor, buckets: int, mul_prev: int,
                    mul_cur: int, vocab: int) -> None:
    """hidden[t] += table[(token before * mul_prev + token * mul_cur) mod buckets]; a sequence's first
    token takes row `buckets`.  The token before a portion's first token comes from `last_token`
    [slots] i32 (one word per request's state slot), which then takes the portion's last token."""
    flush_gemm_chain()
    _cuda_contig("hidden", hidden, torch.float32)
    _cuda_contig("table", table)
    for name, t in (("ids", ids), ("positions", positions), ("seq_index", seq_index), ("cu_seqlens", cu_seqlens),
                    ("state_slots", state_slots), ("last_token", last_token)):
        _cuda_contig(name, t, torch.int32)
    T, H = hidden.shape
    if table.shape != (buckets + 1, H):
        raise KernelError(f"pair_hash_embed: the table must be [{buckets + 1}, {H}], got {tuple(table.shape)}")
    if min(ids.numel(), positions.numel(), seq_index.numel()) < T:
        raise KernelError("pair_hash_embed: ids, positions and seq_index need one entry per token")
    _check("pair_hash_embed", _fn("ts_pair_hash_embed")(
        hidden.data_ptr(), table.data_ptr(), _act_code("table", table), ids.data_ptr(), positions.data_ptr(), seq_index.data_ptr(),
        cu_seqlens.data_ptr(), state_slots.data_ptr(), last_token.data_ptr(), T, H, int(vocab), int(buckets), int(mul_prev),
        int(mul_cur), _stream()))


def rmsnorm_add(branch: torch.Tensor, weight: torch.Tensor, hidden: torch.Tensor, eps: float, rounded: Optional[torch.Tensor] = None) -> None:
    """hidden += branch * rsqrt(mean(branch^2) + eps) * weight in float32 (the norm sits on the
    branch's output); `rounded`, if given, takes the new rows of hidden in its own element type."""
    flush_gemm_chain()
    _cuda_contig("branch", branch)
    _cuda_contig("weight", weight, torch.float32)
    _cuda_contig("hidden", hidden, torch.float32)
    T, H = hidden.shape
    if branch.shape != hidden.shape or weight.numel() != H:
        raise KernelError(f"rmsnorm_add: shapes disagree: branch {tuple(branch.shape)}, hidden {tuple(hidden.shape)}, weight {tuple(weight.shape)}")
    code = 0
    if rounded is not None:
        _cuda_contig("rounded", rounded)
        if rounded.shape != hidden.shape:
            raise KernelError("rmsnorm_add: rounded must have hidden's shape")
        code = _act_code("rounded", rounded)
    _check("rmsnorm_add", _fn("ts_rmsnorm_add")(
        branch.data_ptr(), _act_code("branch", branch), weight.data_ptr(), hidden.data_ptr(), _ptr(rounded), code, T, H, float(eps), _stream()))


def round_rows(rows: torch.Tensor, out: torch.Tensor) -> None:
    """out = rows in out's element type (float32 -> bfloat16 rounds; bfloat16 -> float32 widens)."""
    flush_gemm_chain()
    _cuda_contig("rows", rows)
    _cuda_contig("out", out)
    if out.shape != rows.shape:
        raise KernelError("round_rows: shapes disagree")
    _check("round_rows", _fn("ts_round_rows")(rows.data_ptr(), _act_code("rows", rows), out.data_ptr(), _act_code("out", out), rows.numel(), _stream()))


def branch_norm_add(branch: torch.Tensor, weight: torch.Tensor, scale: Optional[torch.Tensor], hidden: torch.Tensor, eps: float,
                    next_weight: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None, next_eps: Optional[float] = None) -> None:
    """hidden += branch * rsqrt(mean(branch^2) + eps) * weight (* scale, if given) in float32: a sublayer's
    output norm and its per-channel scale on the way back into the stream.  With `next_weight` and
    `out` the norm that reads the stream next runs in the same pass:
    out = hidden * rsqrt(mean(hidden^2) + next_eps) * next_weight, in branch's element type (next_eps: eps unless given)."""
    flush_gemm_chain()
    _cuda_contig("branch", branch)
    _cuda_contig("weight", weight, torch.float32)
    _cuda_contig("hidden", hidden, torch.float32)
    T, H = hidden.shape
    if branch.shape != hidden.shape or weight.numel() != H:
        raise KernelError(f"branch_norm_add: shapes disagree: branch {tuple(branch.shape)}, hidden {tuple(hidden.shape)}, weight {tuple(weight.shape)}")
    if scale is not None:
        _cuda_contig("scale", scale, torch.float32)
        if scale.numel() != H:
            raise KernelError("branch_norm_add: scale must have one entry per channel")
    if (next_weight is None) != (out is None):
        raise KernelError("branch_norm_add: next_weight and out come together")
    code = _act_code("branch", branch)
    if out is not None:
        _cuda_contig("next_weight", next_weight, torch.float32)
        _cuda_contig("out", out, branch.dtype)
        if out.shape != hidden.shape or next_weight.numel() != H:
            raise KernelError("branch_norm_add: out must have hidden's shape and next_weight one entry per channel")
    _check("branch_norm_add", _fn("ts_branch_norm_add")(
        branch.data_ptr(), code, weight.data_ptr(), _ptr(scale), hidden.data_ptr(), _ptr(next_weight), _ptr(out), code, T, H, float(eps),
        float(eps if next_eps is None else next_eps), _stream()))


def stream_add(hidden: torch.Tensor, rows: Optional[torch.Tensor], vector: Optional[torch.Tensor]) -> None:
    """hidden += rows (if given, [T, H] float32) + vector (if given, [H] float32), in float32."""
    flush_gemm_chain()
    _cuda_contig("hidden", hidden, torch.float32)
    T, H = hidden.shape
    if rows is not None:
        _cuda_contig("rows", rows, torch.float32)
        if rows.shape != hidden.shape:
            raise KernelError("stream_add: rows must have hidden's shape")
    if vector is not None:
        _cuda_contig("vector", vector, torch.float32)
        if vector.numel() != H:
            raise KernelError("stream_add: vector must have one entry per channel")
    _check("stream_add", _fn("ts_stream_add")(hidden.data_ptr(), _ptr(rows), _ptr(vector), T, H, _stream()))


def qk_joint_norm_rope_store(qk: torch.Tensor, q_out: torch.Tensor, k_dst: torch.Tensor, v_dst: torch.Tensor,
                             slot_mapping: Optional[torch.Tensor], q_norm_weight: torch.Tensor, k_norm_weight: torch.Tensor, eps: float,
                             cos_sin: Optional[torch.Tensor], num_heads: int, num_kv_heads: int, head_dim: int) -> None:
    """RMS norm over a token's whole q row and whole k row (one mean each over all heads' entries),
    rotate-half rotation of every head's first entries, and the stores: q to q_out [T, nq*d], the
    normed and rotated k to k_dst and the k row as projected to v_dst (cache pools [slots, nkv, d]
    by `slot_mapping` [T] i32, -1 = skip; dense [T, nkv, d] without it).

    qk [T, (nq + nkv) * d] with any row stride; norm weights [nq*d] and [nkv*d] float32; cos_sin
    [T, rot/2, 2] float32 (the step's table) or None for no rotation."""
    flush_gemm_chain()
    nq, nkv, d = int(num_heads), int(num_kv_heads), int(head_dim)
    if not qk.is_cuda or qk.dim() != 2 or qk.stride(1) != 1 or qk.shape[1] != (nq + nkv) * d:
        raise KernelError(f"qk_joint_norm_rope_store: qk must be a CUDA matrix [T, {(nq + nkv) * d}] with unit inner stride, got {tuple(qk.shape)}")
    T = qk.shape[0]
    _cuda_contig("q_out", q_out, qk.dtype)
    _cuda_contig("k_dst", k_dst, qk.dtype)
    _cuda_contig("v_dst", v_dst, qk.dtype)
    _cuda_contig("q_norm_weight", q_norm_weight, torch.float32)
    _cuda_contig("k_norm_weight", k_norm_weight, torch.float32)
    if q_out.numel() != T * nq * d or q_norm_weight.numel() != nq * d or k_norm_weight.numel() != nkv * d:
        raise KernelError("qk_joint_norm_rope_store: q_out or the norm weights do not match the heads")
    for name, c in (("k_dst", k_dst), ("v_dst", v_dst)):
        if tuple(c.shape[-2:]) != (nkv, d):
            raise KernelError(f"qk_joint_norm_rope_store: {name} must end in [{nkv},{d}], got {tuple(c.shape)}")
        if slot_mapping is None and c.numel() < T * nkv * d:
            raise KernelError(f"qk_joint_norm_rope_store: the dense {name} is too small")
    if slot_mapping is not None:
        _cuda_contig("slot_mapping", slot_mapping, torch.int32)
        if slot_mapping.numel() < T:
            raise KernelError("qk_joint_norm_rope_store: slot_mapping is shorter than the batch")
    rot = 0
    if cos_sin is not None:
        _cuda_contig("cos_sin", cos_sin, torch.float32)
        if cos_sin.dim() != 3 or cos_sin.shape[0] < T or cos_sin.shape[2] != 2:
            raise KernelError(f"qk_joint_norm_rope_store: cos_sin must be [T, rot/2, 2], got {tuple(cos_sin.shape)}")
        rot = 2 * cos_sin.shape[1]
        if rot > d:
            raise KernelError(f"qk_joint_norm_rope_store: rotary width {rot} does not fit head_dim {d}")
    _check("qk_joint_norm_rope_store", _fn("ts_qk_joint_norm_rope_store")(
        qk.data_ptr(), _act_code("qk", qk), qk.stride(0), q_out.data_ptr(), k_dst.data_ptr(), v_dst.data_ptr(), _ptr(slot_mapping),
        q_norm_weight.data_ptr(), k_norm_weight.data_ptr(), float(eps), _ptr(cos_sin), rot, T, nq, nkv, d, _stream()))


GLA_MAX_KEY_DIM = 1024
GLA_SEGMENT_TOKENS = 256  # a portion of at least twice as many tokens is cut into segments that run side by side
GLA_MAX_SEGMENTS = 64     # segments of all sequences of a step together (their end states live in scratch)


GLA_ONE_PIECE_CTAS = 2 * 148  # from this many CTAs on, a step's portions run in one piece however long they are


def gla_ctas_per_sequence(num_heads: int, key_dim: int, state_columns: int) -> int:
    """CTAs of the recurrence kernel that one sequence's portion gets when it runs in one piece: heads x
    blocks of value columns (128 threads, of which as many share a column as leave a thread 16 key channels at most)."""
    lanes = 1
    while lanes < 32 and -(-key_dim // lanes) > 16:
        lanes *= 2
    return num_heads * -(-state_columns // (128 // lanes))


def gla_segments(num_seqs: int, max_seqlen: Optional[int], ctas_per_seq: int = 0) -> tuple[int, int]:
    """(segments per sequence, tokens per segment) of a step whose longest portion has `max_seqlen`
    tokens; (1, 0): every portion in one piece.  A function of the batch's size, its longest portion
    and the mixer's sizes (`ctas_per_seq`, gla_ctas_per_sequence) alone: segments shorten the chain of
    a portion's tokens at the price of half as much work again, which pays only while the CTAs of the
    portions in one piece would leave the SMs idle (measured with 64 heads of 128 x 64 and 2,048 tokens:
    256 CTAs 1.19 ms in segments, 1.25 in one piece; 512 CTAs 2.24 against 1.51; 1,024 CTAs 4.38 against 2.92)."""
    if max_seqlen is None or max_seqlen < 2 * GLA_SEGMENT_TOKENS or num_seqs * ctas_per_seq >= GLA_ONE_PIECE_CTAS:
        return 1, 0
    seg_len = GLA_SEGMENT_TOKENS
    while num_seqs * -(-max_seqlen // seg_len) > GLA_MAX_SEGMENTS and seg_len < max_seqlen:
        seg_len *= 2
    segs = -(-max_seqlen // seg_len)
    return (segs, seg_len) if segs > 1 else (1, 0)


def gla_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, z: torch.Tensor, bias: Optional[torch.Tensor], tau: float, q_scale: float,
             state: torch.Tensor, state_slots: torch.Tensor, cu_seqlens: torch.Tensor, out: torch.Tensor, num_seqs: int, num_heads: int,
             key_dim: int, value_dim: int, max_seqlen: Optional[int] = None) -> None:
    """The recurrence of gated linear attention over the step's tokens, sequence by sequence:
    decay = sigmoid(z + bias)^(1/tau) per key channel, S <- diag(decay) S + k v^T, out = S^T (q * q_scale).

    q, k [T, H*d] and v [T, H*e]: views with one common row stride (columns of one product's result);
    z [T, H*d] with its own; bias [H*d] float32 or None; state [slots, H, d, e] float32, read at a
    sequence's slot before its first token of the step and written after its last; state_slots [B],
    cu_seqlens [B+1] int32; out [T, H*e] float32.  Everything but the loads is float32.  Two launches:
    the decays of all tokens and channels once (float32 scratch [T, H*d]), then the recurrence.
    `max_seqlen`: the most tokens a sequence brings; given, long portions are cut into segments that
    run side by side (gla_segments; two launches of the recurrence: every segment's end state and
    decay product from a zero state, then the read-outs from the folded start states).  The sums of a
    token then depend on where its portion began, in the order of float32 rounding."""
    flush_gemm_chain()
    H, d, e = int(num_heads), int(key_dim), int(value_dim)
    if d > GLA_MAX_KEY_DIM:
        raise KernelError(f"gla_scan: at most {GLA_MAX_KEY_DIM} key channels per head, got {d}")
    T = q.shape[0]
    for name, t, width in (("q", q, H * d), ("k", k, H * d), ("v", v, H * e), ("z", z, H * d)):
        if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1 or tuple(t.shape) != (T, width) or t.dtype != q.dtype:
            raise KernelError(f"gla_scan: {name} must be a CUDA matrix [{T}, {width}] of {q.dtype} with unit inner stride, got {tuple(t.shape)} {t.dtype}")
    if not (q.stride(0) == k.stride(0) == v.stride(0)):
        raise KernelError("gla_scan: q, k and v must share one row stride")
    _cuda_contig("state", state, torch.float32)
    _cuda_contig("state_slots", state_slots, torch.int32)
    _cuda_contig("cu_seqlens", cu_seqlens, torch.int32)
    _cuda_contig("out", out, torch.float32)
    if tuple(state.shape[1:]) != (H, d, e) or out.shape != (T, H * e):
        raise KernelError(f"gla_scan: state must be [slots, {H}, {d}, {e}] and out [{T}, {H * e}], got {tuple(state.shape)} and {tuple(out.shape)}")
    if state_slots.numel() < num_seqs or cu_seqlens.numel() < num_seqs + 1:
        raise KernelError("gla_scan: state_slots and cu_seqlens are shorter than the batch")
    if bias is not None:
        _cuda_contig("bias", bias, torch.float32)
        if bias.numel() != H * d:
            raise KernelError("gla_scan: the bias must have one entry per key channel")
    decay = torch.empty((T, H * d), device=q.device, dtype=torch.float32)
    code, stream = _act_code("q", q), _stream()
    _check("gla_scan", _fn("ts_gla_decay")(z.data_ptr(), z.stride(0), code, _ptr(bias), float(tau), decay.data_ptr(), T, H * d, stream))
    segs, seg_len = gla_segments(int(num_seqs), max_seqlen, gla_ctas_per_sequence(H, d, e))
    if segs == 1 and max_seqlen == 1:
        seg_len = 1  # every sequence brings one token at most: the kernel that stages nothing
    scratch = None
    if segs > 1:
        need = int(num_seqs) * segs * H * d * e + int(num_seqs) * segs * H * d + int(num_seqs) * H * d * e
        scratch = torch.empty(need, device=q.device, dtype=torch.float32)
    _check("gla_scan", _fn("ts_gla_scan")(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), code, decay.data_ptr(), float(q_scale), state.data_ptr(),
        state_slots.data_ptr(), cu_seqlens.data_ptr(), out.data_ptr(), int(num_seqs), H, d, e, segs, seg_len, _ptr(scratch), stream))
    if segs > 1:
        global launch_count
        launch_count += 1  # the recurrence ran as two kernels


def gla_norm_gate(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, num_heads: int, value_dim: int, eps: float) -> None:
    """out[t, h] = o[t, h] * rsqrt(mean(o[t, h]^2) + eps) * weight * silu(gate[t, h]) per head of `value_dim`
    entries.  o [T, H*e] float32; gate [T, H*e] (any row stride) and out [T, H*e] in the compute type;
    weight [e] float32, the same for every head."""
    flush_gemm_chain()
    H, e = int(num_heads), int(value_dim)
    _cuda_contig("o", o, torch.float32)
    _cuda_contig("weight", weight, torch.float32)
    _cuda_contig("out", out)
    T = o.shape[0]
    if not gate.is_cuda or gate.dim() != 2 or gate.stride(1) != 1 or tuple(gate.shape) != (T, H * e) or gate.dtype != out.dtype:
        raise KernelError(f"gla_norm_gate: gate must be a CUDA matrix [{T}, {H * e}] of {out.dtype}, got {tuple(gate.shape)} {gate.dtype}")
    if o.shape != (T, H * e) or out.shape != (T, H * e) or weight.numel() != e:
        raise KernelError("gla_norm_gate: shapes disagree")
    _check("gla_norm_gate", _fn("ts_gla_norm_gate")(o.data_ptr(), gate.data_ptr(), gate.stride(0), _act_code("out", out), weight.data_ptr(),
                                                    out.data_ptr(), T, H, e, float(eps), _stream()))



# ---------------------------------------------------------------------------
# the linear recurrence in its general form, and what stands around it in mixers whose decay is one
# number per (token, head)

_SIGNATURES.update({
    "ts_linear_scan": [_c_void_p, _c_void_p, _c_void_p, _c_ll, _c_int, _c_void_p, _c_int, _c_void_p, _c_float, _c_void_p, _c_ll, _c_void_p,
                       _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "ts_rows_dot_f32": [_c_void_p, _c_int, _c_ll, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
    "ts_mlstm_gate_scan": [_c_void_p, _c_void_p, _c_float, _c_void_p, _c_ll, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p],
    "ts_mlstm_norm_gate": [_c_void_p, _c_void_p, _c_void_p, _c_ll, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_float, _c_void_p],
    "ts_ssm_conv": [_c_void_p, _c_int, _c_ll, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_ll, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int,
                    _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p],
    "ts_ssm_conv_state": [_c_void_p, _c_int, _c_ll, _c_int, _c_void_p, _c_ll, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p],
    "ts_ssm_gate_norm": [_c_void_p, _c_void_p, _c_ll, _c_void_p, _c_void_p, _c_ll, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int,
                         _c_float, _c_void_p],
    "ts_scale_rows": [_c_void_p, _c_ll, _c_float, _c_void_p],
    "ts_rope_table": [_c_void_p, _c_void_p, _c_float, _c_int, _c_int, _c_void_p, _c_void_p],
    "ts_qkv_prepare": [_c_void_p, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_float,
                       _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_float, _c_int,
                       _c_void_p],
    "ts_softcap_rows": [_c_void_p, _c_ll, _c_float, _c_void_p],
    "ts_causal_conv": [_c_void_p, _c_int, _c_ll, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_ll, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                       _c_int, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "ts_delta_scan": [_c_void_p, _c_ll, _c_int, _c_int, _c_int, _c_void_p, _c_ll, _c_void_p, _c_void_p, _c_void_p, _c_ll, _c_void_p, _c_void_p,
                      _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_float, _c_int, _c_void_p],
    "ts_gate_rows": [_c_void_p, _c_void_p, _c_ll, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "ts_weighted_sum": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_float, _c_float, _c_float, _c_float, _c_int, _c_void_p, _c_int, _c_ll,
                        _c_void_p],
})


def _matrix_view(name: str, t: torch.Tensor, rows: int, cols: int, dtype: Optional[torch.dtype] = None) -> None:
    if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1 or tuple(t.shape) != (rows, cols) or (dtype is not None and t.dtype != dtype):
        raise KernelError(f"{name} must be a CUDA matrix [{rows}, {cols}]{'' if dtype is None else ' of ' + str(dtype)} with unit inner stride, "
                          f"got {tuple(t.shape)} {t.dtype}")


def linear_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, kscale: Optional[torch.Tensor], q_scale: float,
                state: torch.Tensor, state_slots: torch.Tensor, cu_seqlens: torch.Tensor, out: torch.Tensor, num_seqs: int, num_heads: int,
                groups: int, key_dim: int, value_dim: int, normaliser: bool = False, max_seqlen: Optional[int] = None) -> None:
    """S_t = a_t S_(t-1) + (b_t k_t) v_t^T,  out_t = S_t^T (q_t * q_scale), per head, over the step's tokens
    sequence by sequence, with one decay a_t per (token, head).

    q, k [T, groups*d] (head h reads group h // (H // groups)) and v [T, H*e]: views with one common
    row stride, float32 or bfloat16 (all three alike); decay [T, H] and kscale [T, H] (or None) float32.
    state [slots, n] float32 with n >= H*d*e': a request's [H, d, e'] block stands at the start of its
    row, e' = e + 1 with `normaliser` (the extra column is fed the value 1 in every token, so it holds
    the sum of the decayed b_t k_t, and its read-out arrives as column e of out), else e' = e.
    out [T, H*e'] float32.  Long portions run in segments side by side as in gla_scan."""
    flush_gemm_chain()
    H, G, d, e = int(num_heads), int(groups), int(key_dim), int(value_dim)
    ee = e + 1 if normaliser else e
    if d > GLA_MAX_KEY_DIM:
        raise KernelError(f"linear_scan: at most {GLA_MAX_KEY_DIM} key channels per head, got {d}")
    if G < 1 or H % G:
        raise KernelError(f"linear_scan: {H} heads are no multiple of {G} groups")
    T = q.shape[0]
    _matrix_view("linear_scan: q", q, T, G * d)
    _matrix_view("linear_scan: k", k, T, G * d, q.dtype)
    _matrix_view("linear_scan: v", v, T, H * e, q.dtype)
    if not (q.stride(0) == k.stride(0) == v.stride(0)):
        raise KernelError("linear_scan: q, k and v must share one row stride")
    _cuda_contig("decay", decay, torch.float32)
    if kscale is not None:
        _cuda_contig("kscale", kscale, torch.float32)
    for name, t in (("decay", decay), ("kscale", kscale)):
        if t is not None and tuple(t.shape) != (T, H):
            raise KernelError(f"linear_scan: {name} must be [{T}, {H}], got {tuple(t.shape)}")
    _cuda_contig("state_slots", state_slots, torch.int32)
    _cuda_contig("cu_seqlens", cu_seqlens, torch.int32)
    _cuda_contig("out", out, torch.float32)
    if not state.is_cuda or state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] < H * d * ee:
        raise KernelError(f"linear_scan: state must be float32 [slots, >= {H * d * ee}], got {tuple(state.shape)} {state.dtype}")
    if out.shape != (T, H * ee):
        raise KernelError(f"linear_scan: out must be [{T}, {H * ee}], got {tuple(out.shape)}")
    if state_slots.numel() < num_seqs or cu_seqlens.numel() < num_seqs + 1:
        raise KernelError("linear_scan: state_slots and cu_seqlens are shorter than the batch")
    segs, seg_len = gla_segments(int(num_seqs), max_seqlen, gla_ctas_per_sequence(H, d, ee))
    if segs == 1 and max_seqlen == 1:
        seg_len = 1  # every sequence brings one token at most: the kernel that stages nothing
    scratch = None
    if segs > 1:
        need = int(num_seqs) * segs * H * d * ee + int(num_seqs) * segs * H * d + int(num_seqs) * H * d * ee
        scratch = torch.empty(need, device=q.device, dtype=torch.float32)
    _check("linear_scan", _fn("ts_linear_scan")(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), _act_code("q", q), decay.data_ptr(), 1, _ptr(kscale), float(q_scale),
        state.data_ptr(), state.stride(0), state_slots.data_ptr(), cu_seqlens.data_ptr(), out.data_ptr(), int(num_seqs), H, G, d, e, ee,
        segs, seg_len, _ptr(scratch), _stream()))
    if segs > 1:
        global launch_count
        launch_count += 1  # the recurrence ran as two kernels


def rows_dot_f32(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out[t, r] = x[t] . weight[r] + bias[r] with float32 weights and sums; x [T, W] float32 or
    bfloat16 (any row stride), weight [R, W] float32, out [T, R] float32."""
    flush_gemm_chain()
    _cuda_contig("weight", weight, torch.float32)
    _cuda_contig("out", out, torch.float32)
    T, (R, W) = x.shape[0], weight.shape
    _matrix_view("rows_dot_f32: x", x, T, W)
    if bias is not None:
        _cuda_contig("bias", bias, torch.float32)
    if out.shape != (T, R) or (bias is not None and bias.numel() != R):
        raise KernelError("rows_dot_f32: shapes disagree")
    _check("rows_dot_f32", _fn("ts_rows_dot_f32")(x.data_ptr(), _act_code("x", x), x.stride(0), weight.data_ptr(), _ptr(bias), out.data_ptr(),
                                                  T, R, W, _stream()))


def mlstm_gate_scan(pre: torch.Tensor, cap: float, m_state: torch.Tensor, state_slots: torch.Tensor, cu_seqlens: torch.Tensor, num_seqs: int,
                    num_heads: int, bias: Optional[torch.Tensor] = None) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """From pre [T, 2H] float32 (input-gate rows, then forget-gate rows; `bias` [2H] float32 is added): the running maximum m of the
    gates' logarithms per (token, head), carried in m_state [slots, >= H] (a view whose rows are the
    requests' slots), and what the recurrence needs of it: decay = exp(log_f + m_prev - m) and
    kscale = exp(log_i - m), each [T, H] float32.  Returns (decay, kscale, m)."""
    H = int(num_heads)
    flush_gemm_chain()
    _cuda_contig("pre", pre, torch.float32)
    if bias is not None:
        _cuda_contig("bias", bias, torch.float32)
        if bias.numel() != 2 * H:
            raise KernelError(f"mlstm_gate_scan: bias must have {2 * H} entries, got {bias.numel()}")
    T = pre.shape[0]
    if pre.shape != (T, 2 * H):
        raise KernelError(f"mlstm_gate_scan: pre must be [{T}, {2 * H}], got {tuple(pre.shape)}")
    if not m_state.is_cuda or m_state.dtype != torch.float32 or m_state.dim() != 2 or m_state.stride(1) != 1 or m_state.shape[1] < H:
        raise KernelError("mlstm_gate_scan: m_state must be a float32 view [slots, >= heads]")
    decay = torch.empty((T, H), device=pre.device, dtype=torch.float32)
    kscale = torch.empty_like(decay)
    m = torch.empty_like(decay)
    _check("mlstm_gate_scan", _fn("ts_mlstm_gate_scan")(pre.data_ptr(), _ptr(bias), float(cap), m_state.data_ptr(), m_state.stride(0), state_slots.data_ptr(),
                                                        cu_seqlens.data_ptr(), decay.data_ptr(), kscale.data_ptr(), m.data_ptr(),
                                                        int(num_seqs), H, _stream()))
    return decay, kscale, m


def mlstm_norm_gate(o: torch.Tensor, m: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, num_heads: int,
                    value_dim: int, eps: float) -> None:
    """o [T, H*(e+1)] float32 from linear_scan with its normaliser column; m [T, H]; per head
    h = o[:e] / (max(|o[e]|, exp(-m)) + 1e-6), then h / sqrt(mean(h^2) + eps) * weight[h*e:(h+1)*e] *
    sigmoid(gate) into out [T, H*e] (the compute type, like gate)."""
    H, e = int(num_heads), int(value_dim)
    _cuda_contig("o", o, torch.float32)
    _cuda_contig("m", m, torch.float32)
    _cuda_contig("weight", weight, torch.float32)
    _cuda_contig("out", out)
    T = o.shape[0]
    _matrix_view("mlstm_norm_gate: gate", gate, T, H * e, out.dtype)
    if o.shape != (T, H * (e + 1)) or out.shape != (T, H * e) or weight.numel() != H * e or m.shape != (T, H):
        raise KernelError("mlstm_norm_gate: shapes disagree")
    _check("mlstm_norm_gate", _fn("ts_mlstm_norm_gate")(o.data_ptr(), m.data_ptr(), gate.data_ptr(), gate.stride(0), _act_code("out", out),
                                                        weight.data_ptr(), out.data_ptr(), T, H, e, float(eps), _stream()))


def ssm_conv(xin: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor, conv_state: torch.Tensor, state_slots: torch.Tensor,
             cu_seqlens: torch.Tensor, seq_index: torch.Tensor, num_seqs: int, dt_raw: torch.Tensor, dt_bias: torch.Tensor,
             a_log: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Causal convolution per channel with silu, and the step sizes of a state-space layer.

    xin [T, C] (a view, float32 or bfloat16); taps [C, K] and bias [C] float32 (the last tap weighs the
    current token); conv_state: a float32 view [slots, >= (K-1)*C] whose row holds a request's last
    K - 1 inputs [K-1, C], oldest first (read here for the tokens at a portion's start, and brought up
    to date by a second launch).  dt_raw [T, H] float32, dt_bias, a_log [H] float32.
    Returns (conv [T, C] float32, dt = softplus(dt_raw + dt_bias) [T, H], decay = exp(-exp(a_log) dt) [T, H])."""
    flush_gemm_chain()
    T, C = xin.shape
    K, H = int(taps.shape[1]), int(dt_bias.numel())
    _matrix_view("ssm_conv: xin", xin, T, C)
    for name, t in (("taps", taps), ("bias", bias), ("dt_raw", dt_raw), ("dt_bias", dt_bias), ("a_log", a_log)):
        _cuda_contig(name, t, torch.float32)
    if taps.shape != (C, K) or bias.numel() != C or dt_raw.shape != (T, H) or a_log.numel() != H:
        raise KernelError("ssm_conv: shapes disagree")
    if (not conv_state.is_cuda or conv_state.dtype != torch.float32 or conv_state.dim() != 2 or conv_state.stride(1) != 1
            or conv_state.shape[1] < (K - 1) * C):
        raise KernelError("ssm_conv: conv_state must be a float32 view [slots, >= (taps - 1) * channels]")
    out = torch.empty((T, C), device=xin.device, dtype=torch.float32)
    dt = torch.empty((T, H), device=xin.device, dtype=torch.float32)
    decay = torch.empty_like(dt)
    code, stream = _act_code("xin", xin), _stream()
    _check("ssm_conv", _fn("ts_ssm_conv")(
        xin.data_ptr(), code, xin.stride(0), taps.data_ptr(), bias.data_ptr(), K, conv_state.data_ptr(), conv_state.stride(0),
        state_slots.data_ptr(), cu_seqlens.data_ptr(), seq_index.data_ptr(), out.data_ptr(), T, C, dt_raw.data_ptr(), dt_bias.data_ptr(),
        a_log.data_ptr(), dt.data_ptr(), decay.data_ptr(), H, stream))
    if K > 1:
        _check("ssm_conv", _fn("ts_ssm_conv_state")(xin.data_ptr(), code, xin.stride(0), K, conv_state.data_ptr(), conv_state.stride(0),
                                                    state_slots.data_ptr(), cu_seqlens.data_ptr(), int(num_seqs), C, stream))
    return out, dt, decay


def ssm_gate_norm(o: torch.Tensor, x: torch.Tensor, skip: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, out: torch.Tensor,
                  num_heads: int, value_dim: int, parts: int, eps: float) -> None:
    """y = (o + skip[h] * x) * silu(z), RMS-normed in `parts` equal parts of the row (each by its own root
    mean square), times weight.  o [T, H*e] float32; x [T, H*e] float32 (a view); z (a view) and out
    [T, H*e] in the compute type; skip [H] and weight [H*e] float32."""
    H, e = int(num_heads), int(value_dim)
    T = o.shape[0]
    _cuda_contig("o", o, torch.float32)
    _cuda_contig("skip", skip, torch.float32)
    _cuda_contig("weight", weight, torch.float32)
    _cuda_contig("out", out)
    _matrix_view("ssm_gate_norm: x", x, T, H * e, torch.float32)
    _matrix_view("ssm_gate_norm: z", z, T, H * e, out.dtype)
    if o.shape != (T, H * e) or out.shape != (T, H * e) or weight.numel() != H * e or skip.numel() != H or parts < 1 or (H * e) % parts:
        raise KernelError("ssm_gate_norm: shapes disagree")
    _check("ssm_gate_norm", _fn("ts_ssm_gate_norm")(o.data_ptr(), x.data_ptr(), x.stride(0), skip.data_ptr(), z.data_ptr(), z.stride(0),
                                                    _act_code("out", out), weight.data_ptr(), out.data_ptr(), T, H, e, int(parts), float(eps),
                                                    _stream()))


def scale_rows(x: torch.Tensor, factor: float) -> None:
    """x *= factor in place, float32."""
    flush_gemm_chain()
    _cuda_contig("x", x, torch.float32)
    _check("scale_rows", _fn("ts_scale_rows")(x.data_ptr(), x.numel(), float(factor), _stream()))


def softcap_rows(x: torch.Tensor, cap: float) -> None:
    """x = cap * tanh(x / cap) in place, float32."""
    flush_gemm_chain()
    _cuda_contig("x", x, torch.float32)
    if not cap > 0:
        raise KernelError("softcap_rows: the cap must be positive")
    _check("softcap_rows", _fn("ts_softcap_rows")(x.data_ptr(), x.numel(), float(cap), _stream()))


CONV_ACTIVATIONS = {None: 0, "silu": 1}


def causal_conv(xin: torch.Tensor, taps: torch.Tensor, bias: Optional[torch.Tensor], conv_state: Optional[torch.Tensor], state_slots: torch.Tensor,
                cu_seqlens: torch.Tensor, seq_index: torch.Tensor, num_seqs: int, out: torch.Tensor, activation: Optional[str] = None,
                add_input: bool = False) -> None:
    """A short causal convolution over time on every channel of xin [T, C] (a view of a wider matrix
    is fine): out[t] = act(sum_j taps[j] * x[t - (K-1) + j] + bias), or with `add_input`
    x[t] + that.  taps [K, C] float32, tap by tap (the last row weighs the current token; a checkpoint's
    [C, K] is transposed once at load), bias [C] float32 or None.  conv_state [slots, >= (K-1)*C] float32 (a view with a row stride is fine) holds the last
    K - 1 inputs of every request, oldest first; it is read for the inputs before a portion and then
    brought up to date with the portion's last inputs (K = 1: there is none, and conv_state may be None).
    Sums in float32; xin and out may differ in type."""
    flush_gemm_chain()
    T, C = xin.shape
    K = taps.shape[0]
    _matrix_view("causal_conv: xin", xin, T, C)
    _matrix_view("causal_conv: out", out, T, C)
    _cuda_contig("taps", taps, torch.float32)
    if taps.shape != (K, C):
        raise KernelError(f"causal_conv: taps must be [K, {C}], got {tuple(taps.shape)}")
    if bias is not None:
        _cuda_contig("bias", bias, torch.float32)
    if K > 1 and (conv_state is None or conv_state.dtype != torch.float32 or conv_state.dim() != 2 or conv_state.stride(1) != 1
                  or conv_state.shape[1] < (K - 1) * C):
        raise KernelError(f"causal_conv: the state must be float32 [slots, >= {(K - 1) * C}]")
    state_ptr, state_stride = (None, 0) if K == 1 else (conv_state.data_ptr(), conv_state.stride(0))
    if activation not in CONV_ACTIVATIONS:
        raise KernelError(f"causal_conv: activation must be one of {list(CONV_ACTIVATIONS)}, got {activation!r}")
    _check("causal_conv", _fn("ts_causal_conv")(
        xin.data_ptr(), _act_code("xin", xin), xin.stride(0), taps.data_ptr(), _ptr(bias), K, state_ptr, state_stride,
        state_slots.data_ptr(), cu_seqlens.data_ptr(), seq_index.data_ptr(), out.data_ptr(), _act_code("out", out), out.stride(0), T, C,
        CONV_ACTIVATIONS[activation], 1 if add_input else 0, _stream()))


DELTA_MAX_KEY_DIM = 1024
# TS_DELTA_LANES (for measurements): lanes that share a value column of the delta rule's state (a power of two up to 32);
# unset or 0: the kernel's own choice by the key width
DELTA_LANES = int(_os.environ.get("TS_DELTA_LANES", "0"))


def delta_scan(x: torch.Tensor, q_off: int, k_off: int, v_off: int, gates: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor,
               state: torch.Tensor, state_slots: torch.Tensor, cu_seqlens: torch.Tensor, out: torch.Tensor, num_seqs: int, num_heads: int,
               num_qk_heads: int, key_dim: int, value_dim: int, q_scale: float, unit_eps: float) -> None:
    """The gated delta rule over the tokens of every sequence, in order (csrc/delta_rule.cu).  x [T, n]
    float32 holds q (columns q_off.., num_qk_heads * key_dim), k (k_off..) and v (v_off.., num_heads *
    value_dim); q and k are brought to unit length per head here and q is multiplied by q_scale.
    gates [T, 2 * heads] float32: the raw write-strength rows, then the raw decay rows (beta = sigmoid,
    decay = exp(-exp(a_log) * softplus(raw + dt_bias))).  state [slots, >= heads * value_dim * key_dim]
    float32 (a view with a row stride is fine), one head after the other, value column by value column;
    out [T, heads * value_dim] float32."""
    flush_gemm_chain()
    H, G, d, e = int(num_heads), int(num_qk_heads), int(key_dim), int(value_dim)
    T = x.shape[0]
    if not x.is_cuda or x.dtype != torch.float32 or x.dim() != 2 or x.stride(1) != 1:
        raise KernelError("delta_scan: x must be a float32 CUDA matrix with unit inner stride")
    if max(q_off, k_off) + G * d > x.shape[1] or v_off + H * e > x.shape[1]:
        raise KernelError("delta_scan: the column ranges do not fit x")
    _matrix_view("delta_scan: gates", gates, T, 2 * H, torch.float32)
    _cuda_contig("a_log", a_log, torch.float32)
    _cuda_contig("dt_bias", dt_bias, torch.float32)
    _cuda_contig("out", out, torch.float32)
    if a_log.numel() != H or dt_bias.numel() != H or out.shape != (T, H * e):
        raise KernelError("delta_scan: a_log and dt_bias need one entry per head, out must be [T, heads * value_dim]")
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] < H * d * e:
        raise KernelError(f"delta_scan: the state must be float32 [slots, >= {H * d * e}], got {tuple(state.shape)}")
    if d > DELTA_MAX_KEY_DIM or H % G:
        raise KernelError(f"delta_scan: key_dim at most {DELTA_MAX_KEY_DIM}, heads a multiple of the q/k heads")
    _check("delta_scan", _fn("ts_delta_scan")(
        x.data_ptr(), x.stride(0), int(q_off), int(k_off), int(v_off), gates.data_ptr(), gates.stride(0), a_log.data_ptr(), dt_bias.data_ptr(),
        state.data_ptr(), state.stride(0), state_slots.data_ptr(), cu_seqlens.data_ptr(), out.data_ptr(), int(num_seqs), H, G, d, e,
        float(q_scale), float(unit_eps), DELTA_LANES, _stream()))


WEIGHTED_SUM_MAX_INPUTS = 4


def weighted_sum(inputs: "list[torch.Tensor]", scales: "list[float]", out: torch.Tensor) -> None:
    """out = sum_j scales[j] * inputs[j], summed in float32 and rounded once; up to four inputs of
    out's shape and type."""
    flush_gemm_chain()
    if not 1 <= len(inputs) <= WEIGHTED_SUM_MAX_INPUTS or len(inputs) != len(scales):
        raise KernelError(f"weighted_sum: one to {WEIGHTED_SUM_MAX_INPUTS} inputs with a scale each")
    _cuda_contig("out", out)
    for t in inputs:
        _cuda_contig("input", t, out.dtype)
        if t.shape != out.shape:
            raise KernelError("weighted_sum: shapes disagree")
    ptrs = [t.data_ptr() for t in inputs] + [None] * (4 - len(inputs))
    sc = [float(x) for x in scales] + [0.0] * (4 - len(inputs))
    _check("weighted_sum", _fn("ts_weighted_sum")(*ptrs, *sc, len(inputs), out.data_ptr(), _act_code("out", out), out.numel(), _stream()))


# ---------------------------------------------------------------------------
# between a stacked q/k/v projection and attention, for mixers with biases, a rotation with a
# magnitude, a unit norm after the rotation, or values of another width than keys

QKV_PREPARE_MAX_DIM = 512


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, magnitude: float, num_tokens: int) -> torch.Tensor:
    """[num_tokens, len(inv_freq), 2] float32: magnitude * (cos, sin)(positions[t] * inv_freq[j]), the
    angle formed in float64 from float64 frequencies."""
    _cuda_contig("positions", positions, torch.int32)
    _cuda_contig("inv_freq", inv_freq, torch.float64)
    if positions.numel() < num_tokens:
        raise KernelError("rope_table: positions are shorter than the tokens")
    half = inv_freq.numel()
    out = torch.empty((num_tokens, half, 2), device=positions.device, dtype=torch.float32)
    _check("rope_table", _fn("ts_rope_table")(positions.data_ptr(), inv_freq.data_ptr(), float(magnitude), num_tokens, half, out.data_ptr(),
                                              _stream()))
    return out


def qkv_prepare(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, q_bias: Optional[torch.Tensor], k_bias: Optional[torch.Tensor],
                v_bias: Optional[torch.Tensor], table: Optional[torch.Tensor], unit_norm: bool, eps: float, q_out: torch.Tensor,
                k_dst: Optional[torch.Tensor], v_dst: Optional[torch.Tensor], slot_mapping: Optional[torch.Tensor], num_heads: int,
                num_kv_heads: int, key_dim: int, value_dim: int, padded_dim: int, positions: Optional[torch.Tensor] = None,
                query_temperature: Optional[tuple[float, int]] = None) -> None:
    """Queries, keys and values of a step out of one projection's result `proj` [T, n] (columns q_off..,
    k_off.., v_off..): biases [heads*dim] float32 (or None), rotation of the first 2*table.shape[1]
    entries of every q and k head by the table's (cos, sin) (rope_table; None: no rotation), then with
    `unit_norm` q and k heads divided by sqrt(mean(x^2) + eps).  q_out [T, nq, D]; keys and values go to
    k_dst / v_dst [slots, nkv, D] at slot_mapping[t] (None: row t; a negative slot: not kept), padded with
    zeros from their own width to D = padded_dim.  k_dst None: only the queries are made.
    query_temperature = (coef, every) with the tokens' positions: query heads are multiplied by
    1 + coef * ln(floor((position + 1) / every) + 1)."""
    flush_gemm_chain()
    qt_coef, qt_every = (0.0, 0) if query_temperature is None else (float(query_temperature[0]), int(query_temperature[1]))
    if qt_every:
        if qt_every < 1 or positions is None:
            raise KernelError("qkv_prepare: a query temperature needs the positions and a positive step")
        _cuda_contig("positions", positions, torch.int32)
        if positions.numel() < proj.shape[0]:
            raise KernelError("qkv_prepare: positions are shorter than the tokens")
    nq, nkv, d, e, D = int(num_heads), int(num_kv_heads), int(key_dim), int(value_dim), int(padded_dim)
    T = proj.shape[0]
    if not proj.is_cuda or proj.dim() != 2 or proj.stride(1) != 1:
        raise KernelError("qkv_prepare: proj must be a CUDA matrix with unit inner stride")
    if D > QKV_PREPARE_MAX_DIM or D < max(d, e):
        raise KernelError(f"qkv_prepare: heads of {d} / {e} entries padded to {D}: at most {QKV_PREPARE_MAX_DIM}, at least the wider of the two")
    _cuda_contig("q_out", q_out, proj.dtype)
    if q_out.numel() != T * nq * D:
        raise KernelError("qkv_prepare: q_out must be [T, heads, padded_dim]")
    for name, t in (("q_bias", q_bias), ("k_bias", k_bias), ("v_bias", v_bias)):
        if t is not None:
            _cuda_contig(name, t, torch.float32)
    rot = 0
    if table is not None:
        _cuda_contig("table", table, torch.float32)
        if table.dim() != 3 or table.shape[0] < T or table.shape[2] != 2 or 2 * table.shape[1] > d:
            raise KernelError(f"qkv_prepare: the table must be [T, rot/2, 2] with rot <= {d}, got {tuple(table.shape)}")
        rot = 2 * table.shape[1]
    kv_heads = nkv
    if k_dst is None:
        kv_heads = 0
    else:
        _cuda_contig("k_dst", k_dst, proj.dtype)
        _cuda_contig("v_dst", v_dst, proj.dtype)
        if tuple(k_dst.shape[-2:]) != (nkv, D) or tuple(v_dst.shape[-2:]) != (nkv, D):
            raise KernelError(f"qkv_prepare: k_dst and v_dst must end in [{nkv}, {D}], got {tuple(k_dst.shape)} and {tuple(v_dst.shape)}")
    if slot_mapping is not None:
        _cuda_contig("slot_mapping", slot_mapping, torch.int32)
    _check("qkv_prepare", _fn("ts_qkv_prepare")(
        proj.data_ptr(), _act_code("proj", proj), proj.stride(0), int(q_off), int(k_off), int(v_off), _ptr(q_bias), _ptr(k_bias), _ptr(v_bias),
        _ptr(table), rot, 1 if unit_norm else 0, float(eps), q_out.data_ptr(), _ptr(k_dst), _ptr(v_dst), _ptr(slot_mapping), T, nq, kv_heads,
        d, e, D, _ptr(positions) if qt_every else None, qt_coef, qt_every, _stream()))


def gate_rows(a: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor, num_heads: int, value_dim: int, padded_dim: int) -> None:
    """out[t, h*e + i] = a[t, h, i] * sigmoid(gate[t, h*e + i]); a [T, H, D] with D >= e (the entries
    beyond e are dropped); gate None: the compaction alone."""
    H, e, D = int(num_heads), int(value_dim), int(padded_dim)
    _cuda_contig("a", a)
    _cuda_contig("out", out, a.dtype)
    T = out.shape[0]
    if a.numel() != T * H * D or out.shape != (T, H * e):
        raise KernelError("gate_rows: shapes disagree")
    if gate is not None:
        _matrix_view("gate_rows: gate", gate, T, H * e, a.dtype)
    _check("gate_rows", _fn("ts_gate_rows")(a.data_ptr(), _ptr(gate), 0 if gate is None else gate.stride(0), _act_code("a", a), out.data_ptr(),
                                            T, H, e, D, _stream()))


ROTARY_PAIRINGS = {"half": 0, "neighbours": 1}
LATENT_SIMPLE_MAX_KEY_DIM = 1024


def latent_prepare(proj: Optional[torch.Tensor], q_off: int, kv_off: int, gate_off: int, q_abs: torch.Tensor, cache: Optional[torch.Tensor],
                   slot_mapping: Optional[torch.Tensor], positions: torch.Tensor, latent_weight: Optional[torch.Tensor], eps: float,
                   inv_freq: Optional[torch.Tensor], rot_dims: int, pairing: str, gates: Optional[torch.Tensor], num_heads: int,
                   nope_dim: int, rot_dim: int, rank: int, magnitude: float = 1.0, q_src: Optional[torch.Tensor] = None) -> None:
    """What follows the stacked projection of a latent attention layer, per token: the latent (columns
    kv_off .. kv_off+rank of `proj`) RMS-normed with `latent_weight`, the key part behind it and
    every head's rotated query part turned by the token's position, [latent ; key part] stored in
    `cache` [slots, rank+rot] at slot_mapping[t] (-1 or no mapping: not stored), the rotated query
    parts written to q_abs[t, head, rank:], and gates[t, head] = sigmoid(proj[t, gate_off+head]).
    Cosines and sines are multiplied by `magnitude`.  `q_src` [T, heads*(nope+rot)]: the queries come
    from this tensor instead of proj's columns from q_off on.  kv_off < 0: the layer has no latent of
    its own (it reads rows that another layer cached): only the queries are prepared, and `proj` may
    then be None."""
    flush_gemm_chain()
    H, dn, dr = num_heads, nope_dim, rot_dim
    if q_src is not None:
        _cuda_contig("q_src", q_src, q_abs.dtype)
        if q_src.dim() != 2 or q_src.shape[1] != H * (dn + dr):
            raise KernelError(f"latent_prepare: q_src must be [T, {H * (dn + dr)}], got {tuple(q_src.shape)}")
    if proj is None:
        if q_src is None or kv_off >= 0 or gates is not None or cache is not None:
            raise KernelError("latent_prepare: without a projection only queries from q_src are prepared")
        T, ld = q_src.shape[0], 0
    else:
        _cuda_contig("proj", proj, q_abs.dtype)
        T, ld = proj.shape
    _cuda_contig("q_abs", q_abs)
    _cuda_contig("positions", positions, torch.int32)
    if kv_off >= 0:
        _cuda_contig("latent_weight", latent_weight, torch.float32)
    elif cache is not None or slot_mapping is not None:
        raise KernelError("latent_prepare: a layer without a latent of its own stores nothing")
    if q_abs.numel() != T * H * (rank + dr):
        raise KernelError(f"latent_prepare: q_abs must hold [{T}, {H}, {rank + dr}], got {tuple(q_abs.shape)}")
    if (q_src is None and q_off + H * (dn + dr) > ld) or (kv_off >= 0 and kv_off + rank + dr > ld) or (gates is not None and gate_off + H > ld):
        raise KernelError("latent_prepare: the column ranges do not fit the projection's width")
    if slot_mapping is not None:
        if cache is None:
            raise KernelError("latent_prepare: a slot mapping needs the cache")
        _cuda_contig("cache", cache, q_abs.dtype)
        _cuda_contig("slot_mapping", slot_mapping, torch.int32)
        if cache.shape[-1] != rank + dr or slot_mapping.numel() < T:
            raise KernelError(f"latent_prepare: cache rows must be {rank + dr} wide and slot_mapping hold {T} entries")
    if gates is not None:
        _cuda_contig("gates", gates, torch.float32)
        if gates.numel() != T * H:
            raise KernelError("latent_prepare: gates must be [T, heads]")
    if rot_dims:
        if inv_freq is None:
            raise KernelError("latent_prepare: a rotation needs its inverse frequencies")
        _cuda_contig("inv_freq", inv_freq, torch.float32)
        if inv_freq.numel() != rot_dims // 2 or rot_dims > dr or rot_dims % 2:
            raise KernelError(f"latent_prepare: {rot_dims} rotated entries of {dr} need {rot_dims // 2} frequencies")
    _check("latent_prepare", _fn("ts_latent_prepare")(
        _ptr(proj), _act_code("q_abs", q_abs), ld, int(q_off), int(kv_off), int(gate_off), q_abs.data_ptr(), _ptr(cache),
        _ptr(slot_mapping), positions.data_ptr(), _ptr(latent_weight), float(eps), _ptr(inv_freq), int(rot_dims),
        ROTARY_PAIRINGS[pairing], _ptr(gates), T, H, dn, dr, int(rank), float(magnitude), _ptr(q_src),
        0 if q_src is None else q_src.stride(0), _stream()))


def latent_attention_simple(q_abs: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, gates: Optional[torch.Tensor],
                            positions: torch.Tensor, seq_index: torch.Tensor, block_table: torch.Tensor, page_size: int,
                            num_heads: int, rank: int, rot_dim: int, scale: float, window: int = 0) -> None:
    """Causal attention of absorbed queries q_abs [T, H, rank+rot] over cached rows [pages, page,
    rank+rot] on CUDA cores: out [T, H, rank] = softmax(q_abs . row * scale) @ row[:rank], times
    gates[t, h] if given.  Float32 or bfloat16; scores, softmax and sums in float32."""
    flush_gemm_chain()
    _cuda_contig("q_abs", q_abs)
    _cuda_contig("cache", cache, q_abs.dtype)
    _cuda_contig("out", out, q_abs.dtype)
    for name, t in (("positions", positions), ("seq_index", seq_index), ("block_table", block_table)):
        _cuda_contig(name, t, torch.int32)
    T = q_abs.shape[0]
    H, D = num_heads, rank + rot_dim
    if D > LATENT_SIMPLE_MAX_KEY_DIM:
        raise KernelError(f"latent_attention_simple: rank + rotated width must be <= {LATENT_SIMPLE_MAX_KEY_DIM}, got {D}")
    if q_abs.numel() != T * H * D or out.numel() != T * H * rank:
        raise KernelError("latent_attention_simple: q_abs / out do not match [T, heads, rank(+rot)]")
    if tuple(cache.shape[-2:]) != (page_size, D):
        raise KernelError(f"latent_attention_simple: the cache must be [pages, {page_size}, {D}], got {tuple(cache.shape)}")
    if gates is not None:
        _cuda_contig("gates", gates, torch.float32)
    if block_table.dim() != 2 or positions.numel() < T or seq_index.numel() < T:
        raise KernelError("latent_attention_simple: block_table must be [B, max_blocks]; positions and seq_index need T entries")
    _check("latent_attention_simple", _fn("ts_latent_attention_simple")(
        q_abs.data_ptr(), cache.data_ptr(), _act_code("q_abs", q_abs), out.data_ptr(), _ptr(gates), positions.data_ptr(),
        seq_index.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size, T, H, int(rank), int(rot_dim), float(scale),
        int(window), _stream()))


def gelu_tanh(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = z/2 * (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))) element by element (out may be x)."""
    flush_gemm_chain()
    _cuda_contig("x", x)
    _cuda_contig("out", out, x.dtype)
    if out.shape != x.shape:
        raise KernelError("gelu_tanh: shapes disagree")
    _check("gelu_tanh", _fn("ts_gelu_tanh")(x.data_ptr(), out.data_ptr(), _act_code("x", x), x.numel(), _stream()))


def capped_glu(gate_up: torch.Tensor, out: torch.Tensor, limit: float, alpha: float) -> None:
    """out = a * sigmoid(alpha a) * (b + 1), a = min(gate, limit), b = clamp(up, -limit, limit);
    gate_up [T, 2I] holds all gates and then all ups, out [T, I]."""
    flush_gemm_chain()
    _cuda_contig("gate_up", gate_up)
    _cuda_contig("out", out, gate_up.dtype)
    T, I = out.shape
    if gate_up.shape != (T, 2 * I):
        raise KernelError(f"capped_glu: gate_up {tuple(gate_up.shape)} does not match out {tuple(out.shape)}")
    _check("capped_glu", _fn("ts_capped_glu")(gate_up.data_ptr(), out.data_ptr(), _act_code("out", out), T, I, float(limit), float(alpha), _stream()))


def gelu_gate_rows(x: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, col0: int) -> None:
    """x[t, j] = gelu_tanh(x[t, j]) * table[ids[t], col0 + j], in place.  x [T, D], table [V, >= col0 + D]."""
    flush_gemm_chain()
    _cuda_contig("x", x)
    _cuda_contig("table", table, x.dtype)
    _cuda_contig("ids", ids, torch.int32)
    T, D = x.shape
    if ids.numel() < T or col0 < 0 or col0 + D > table.shape[1]:
        raise KernelError(f"gelu_gate_rows: columns {col0}..{col0 + D} of a table {tuple(table.shape)} for {T} tokens")
    _check("gelu_gate_rows", _fn("ts_gelu_gate_rows")(
        x.data_ptr(), table.data_ptr(), _act_code("x", x), ids.data_ptr(), T, D, table.shape[1], int(col0), table.shape[0], _stream()))


MOE_ROW_TILE = 64
MOE_MAX_EXPERTS = 4096


ROUTER_SCORES = {"sigmoid": 0, "softmax_chosen": 1, "softmax_all": 2}


def _router_bias(name: str, bias: Optional[torch.Tensor], E: int) -> Optional[int]:
    if bias is None:
        return None
    _cuda_contig("bias", bias, torch.float32)
    if bias.numel() != E:
        raise KernelError(f"{name}: the bias must have one entry per expert ({E}), got {tuple(bias.shape)}")
    return bias.data_ptr()


def router_topk(logits: torch.Tensor, top: int, renormalize: bool, ids: torch.Tensor, weights: torch.Tensor,
                bias: Optional[torch.Tensor] = None, score: str = "sigmoid", correction: Optional[torch.Tensor] = None) -> None:
    """Per row of float32 logits [T, E] (+ bias [E], if given): the `top` experts with the largest
    logits into ids [T, top] i32 and their weights into weights [T, top] f32.  score "sigmoid": the
    weights are sigmoid(logit) (divided by their sum if `renormalize`); "softmax_chosen": the softmax
    over the chosen logits alone; "softmax_all": the scores are the softmax over all E logits, the
    `top` largest of score + correction [E] are chosen, and the weights are the scores themselves."""
    flush_gemm_chain()
    _cuda_contig("logits", logits, torch.float32)
    _cuda_contig("ids", ids, torch.int32)
    _cuda_contig("weights", weights, torch.float32)
    T, E = logits.shape
    if not 0 < top <= E or ids.numel() != T * top or weights.numel() != T * top:
        raise KernelError(f"router_topk: top {top} of {E} experts, ids {tuple(ids.shape)}, weights {tuple(weights.shape)}")
    _check("router_topk", _fn("ts_router_topk")(logits.data_ptr(), _router_bias("router_topk", bias, E), T, E, int(top),
                                                int(bool(renormalize)), ROUTER_SCORES[score], ids.data_ptr(), weights.data_ptr(),
                                                _router_correction("router_topk", correction, E, score), _stream()))


def _router_correction(name: str, correction: Optional[torch.Tensor], E: int, score: str) -> Optional[int]:
    if correction is not None and score != "softmax_all":
        raise KernelError(f"{name}: a correction of the choice comes with the scores 'softmax_all' only")
    return _router_bias(name, correction, E)


def router(rows: torch.Tensor, router_weight: torch.Tensor, top: int, renormalize: bool, ids: torch.Tensor, weights: torch.Tensor,
           bias: Optional[torch.Tensor] = None, score: str = "sigmoid", correction: Optional[torch.Tensor] = None) -> None:
    """Logits and choice in one kernel: rows [T, W] (float32, or bfloat16 widened on the fly) against
    router_weight [E, W] float32 with float32 sums (+ bias [E] float32, if given), then as router_topk."""
    flush_gemm_chain()
    _cuda_contig("rows", rows)
    _cuda_contig("router_weight", router_weight, torch.float32)
    _cuda_contig("ids", ids, torch.int32)
    _cuda_contig("weights", weights, torch.float32)
    T, W = rows.shape
    E = router_weight.shape[0]
    if router_weight.shape[1] != W or not 0 < top <= E or ids.numel() != T * top or weights.numel() != T * top:
        raise KernelError(f"router: rows {tuple(rows.shape)}, router {tuple(router_weight.shape)}, top {top}, ids {tuple(ids.shape)}")
    _check("router", _fn("ts_router")(rows.data_ptr(), _act_code("rows", rows), router_weight.data_ptr(), _router_bias("router", bias, E),
                                      T, W, E, int(top), int(bool(renormalize)), ROUTER_SCORES[score], ids.data_ptr(), weights.data_ptr(),
                                      _router_correction("router", correction, E, score), _stream()))


# TS_MOE_MMA=0 (for measurements): bfloat16 expert products on CUDA cores too.
MOE_MMA = _os.environ.get("TS_MOE_MMA", "1") != "0"


def moe_on_tensor_cores(dtype: torch.dtype, *inner_widths: int) -> bool:
    """Whether the expert products of these inner widths run on the tensor-core kernels."""
    return MOE_MMA and dtype == torch.bfloat16 and all(k % 8 == 0 for k in inner_widths)


_moe_mma_tiles: Optional[tuple[int, int]] = None
MOE_FEW_ROWS_PER_EXPERT = 12  # up to this many pairs per expert on average the short row tiles are planned


def moe_row_tile(tensor_cores: bool, pairs: int = 0, num_experts: int = 1) -> int:
    """Places per row tile of the expert products' kernels: what a plan is made for.  The tensor-core
    kernels come in two shapes, for many rows per expert and for few (a function of the token count
    alone, so a captured step keeps its shape)."""
    global _moe_mma_tiles
    if not tensor_cores:
        return MOE_ROW_TILE
    if _moe_mma_tiles is None:
        fn = library().ts_moe_mma_row_tile
        fn.argtypes, fn.restype = [_c_int], _c_int
        _moe_mma_tiles = (int(fn(0)), int(fn(1)))
    return _moe_mma_tiles[1] if pairs <= MOE_FEW_ROWS_PER_EXPERT * num_experts else _moe_mma_tiles[0]


def moe_plan(ids: torch.Tensor, num_experts: int, tile_rows: int = MOE_ROW_TILE) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, int]:
    """Sorts the (token, choice) pairs of ids [T, top] by expert on the device.  Returns offsets
    [E+1] (expert e's places are offsets[e]..offsets[e+1]), tile_offsets [E+1] (its first row tile of
    `tile_rows` places), order [T*top] (place -> pair index token*top + choice), and tile_rows."""
    flush_gemm_chain()
    _cuda_contig("ids", ids, torch.int32)
    if num_experts > MOE_MAX_EXPERTS:
        raise KernelError(f"moe_plan: at most {MOE_MAX_EXPERTS} experts, got {num_experts}")
    P = ids.numel()
    plan = torch.empty(2 * (num_experts + 1) + P, dtype=torch.int32, device=ids.device)
    offsets, tile_offsets, order = plan[: num_experts + 1], plan[num_experts + 1 : 2 * (num_experts + 1)], plan[2 * (num_experts + 1) :]
    _check("moe_plan", _fn("ts_moe_plan")(ids.data_ptr(), P, int(num_experts), int(tile_rows), offsets.data_ptr(), tile_offsets.data_ptr(),
                                          order.data_ptr(), _stream()))
    return offsets, tile_offsets, order, int(tile_rows)


def _moe_path(name: str, plan, dtype: torch.dtype, *inner_widths: int) -> bool:
    """True: the tensor-core kernel; the plan's row tile decides, and must suit the kernel it names."""
    if plan[3] == MOE_ROW_TILE:
        return False
    if moe_on_tensor_cores(dtype, *inner_widths):
        moe_row_tile(True)
        if plan[3] in _moe_mma_tiles:
            return True
    raise KernelError(f"{name}: the plan was made for row tiles of {plan[3]}, which no kernel for {dtype} and inner widths {inner_widths} takes")


MOE_ACTIVATIONS = {"capped_glu": 0, "swiglu": 1, "gelu": 2}  # "gelu": experts without a gate matrix, W_down gelu_erf(W_up x)


def moe_gate_up(x: torch.Tensor, pair_weight: torch.Tensor, plan: tuple, gate: Optional[torch.Tensor],
                up: torch.Tensor, act: torch.Tensor, top: int, limit: float, alpha: float, activation: str = "capped_glu") -> None:
    """For every pair, in the plan's order: act[place] = activation(gate_e (w x[token]), up_e (w x[token])), where
    activation is "capped_glu" (with `limit` and `alpha`) or "swiglu" (silu(gate) * up); or, for experts
    without a gate matrix (`gate` None, activation "gelu"), act[place] = gelu_erf(up_e (w x[token])).
    x [T, K]; pair_weight [T*top] f32; gate, up [E, I, K]; act [T*top, I]."""
    flush_gemm_chain()
    offsets, tile_offsets, order, _ = plan
    _cuda_contig("x", x)
    if (gate is None) != (activation == "gelu"):
        raise KernelError("moe_gate_up: the activation 'gelu' comes without a gate matrix, the gated ones with one")
    if gate is None:
        gate_ptr = None
    else:
        _cuda_contig("gate", gate, x.dtype)
        gate_ptr = gate.data_ptr()
    _cuda_contig("up", up, x.dtype)
    _cuda_contig("act", act, x.dtype)
    _cuda_contig("pair_weight", pair_weight, torch.float32)
    T, K = x.shape
    E, I, K2 = up.shape
    P = T * top
    if K2 != K or (gate is not None and up.shape != gate.shape) or act.shape != (P, I) or pair_weight.numel() != P or order.numel() != P:
        raise KernelError(f"moe_gate_up: shapes disagree: x {tuple(x.shape)}, up {tuple(up.shape)}, act {tuple(act.shape)}")
    if _moe_path("moe_gate_up", plan, x.dtype, K):
        _check("moe_gate_up", _fn("ts_moe_gate_up_mma")(
            x.data_ptr(), pair_weight.data_ptr(), order.data_ptr(), offsets.data_ptr(), tile_offsets.data_ptr(), gate_ptr,
            up.data_ptr(), act.data_ptr(), P, E, K, I, int(top), float(limit), float(alpha), MOE_ACTIVATIONS[activation], plan[3], _stream()))
        return
    _check("moe_gate_up", _fn("ts_moe_gate_up")(
        x.data_ptr(), _act_code("x", x), pair_weight.data_ptr(), order.data_ptr(), offsets.data_ptr(), tile_offsets.data_ptr(),
        gate_ptr, up.data_ptr(), act.data_ptr(), P, E, K, I, int(top), float(limit), float(alpha), MOE_ACTIVATIONS[activation], _stream()))


def moe_down(act: torch.Tensor, plan: tuple, down: torch.Tensor, pair_out: torch.Tensor) -> None:
    """pair_out[pair] = down_e act[place] for every place of the plan.  act [P, I]; down [E, N, I]; pair_out [P, N]."""
    flush_gemm_chain()
    offsets, tile_offsets, order, _ = plan
    _cuda_contig("act", act)
    _cuda_contig("down", down, act.dtype)
    _cuda_contig("pair_out", pair_out, act.dtype)
    P, I = act.shape
    E, N, I2 = down.shape
    if I2 != I or pair_out.shape != (P, N) or order.numel() != P:
        raise KernelError(f"moe_down: shapes disagree: act {tuple(act.shape)}, down {tuple(down.shape)}, pair_out {tuple(pair_out.shape)}")
    if _moe_path("moe_down", plan, act.dtype, I):
        _check("moe_down", _fn("ts_moe_down_mma")(
            act.data_ptr(), order.data_ptr(), offsets.data_ptr(), tile_offsets.data_ptr(), down.data_ptr(), pair_out.data_ptr(), P, E, I, N,
            plan[3], _stream()))
        return
    _check("moe_down", _fn("ts_moe_down")(
        act.data_ptr(), _act_code("act", act), order.data_ptr(), offsets.data_ptr(), tile_offsets.data_ptr(), down.data_ptr(),
        pair_out.data_ptr(), P, E, I, N, _stream()))


def moe_combine(pair_out: torch.Tensor, shared: Optional[torch.Tensor], out: torch.Tensor, top: int,
                pair_weight: Optional[torch.Tensor] = None, ids: Optional[torch.Tensor] = None, num_experts: int = 0,
                x: Optional[torch.Tensor] = None) -> None:
    """out[t] = sum of pair_out[t*top .. t*top+top] (each times pair_weight[pair] if given) (+ shared[t]),
    summed in float32.  With `ids` [T, top] i32, `num_experts` and the experts' input rows `x` [T, N], a
    pair whose chosen index is num_experts or more is an identity expert: x[t] stands in for its row of
    pair_out (which nothing has written)."""
    flush_gemm_chain()
    _cuda_contig("pair_out", pair_out)
    _cuda_contig("out", out, pair_out.dtype)
    T, N = out.shape
    if pair_out.shape != (T * top, N):
        raise KernelError(f"moe_combine: pair_out {tuple(pair_out.shape)} does not match out {tuple(out.shape)} with {top} choices")
    if shared is not None:
        _cuda_contig("shared", shared, out.dtype)
        if shared.shape != out.shape:
            raise KernelError("moe_combine: shared must have out's shape")
    if pair_weight is not None:
        _cuda_contig("pair_weight", pair_weight, torch.float32)
        if pair_weight.numel() != T * top:
            raise KernelError("moe_combine: one weight per pair is needed")
    if ids is not None:
        _cuda_contig("ids", ids, torch.int32)
        if x is None or ids.numel() != T * top:
            raise KernelError("moe_combine: identity experts need the chosen indices of every pair and the input rows")
        _cuda_contig("x", x, out.dtype)
        if x.shape != out.shape:
            raise KernelError("moe_combine: x must have out's shape")
    _check("moe_combine", _fn("ts_moe_combine")(pair_out.data_ptr(), _ptr(shared), out.data_ptr(), _ptr(pair_weight), _act_code("out", out),
                                                T, N, int(top), _ptr(ids), int(num_experts), _ptr(x) if ids is not None else None, _stream()))


# ---------------------------------------------------------------------------
# tensor-core latent attention (one library per (rank, rotated width))

LATENT_MMA_MAX_SPLITS = 64
_latent_mma_libs: dict[tuple[int, int], tuple] = {}
_sm_counts: dict[int, int] = {}


def _sm_count(device: torch.device) -> int:
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _sm_counts:
        _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _sm_counts[index]


def latent_attention_mma_supported(rank: int, rot_dim: int) -> bool:
    """Sizes the tensor-core kernel is compiled for: multiples of 16, and tiles of 32 query rows and
    2 x 64 cached rows that fit an SM's shared memory."""
    if rank <= 0 or rank % 16 or rot_dim % 16 or rot_dim < 0:
        return False
    row = (rank + rot_dim + 8) * 2
    return (32 + 2 * 64) * row + 2 * 16 * 72 * 2 + 1024 <= 227 * 1024


def _latent_mma_fns(rank: int, rot_dim: int):
    key = (rank, rot_dim)
    fns = _latent_mma_libs.get(key)
    if fns is None:
        lib = _build.load_variant("latent_attention_mma", {"TS_LAT_RANK": rank, "TS_LAT_ROT": rot_dim})
        fn = lib.ts_latent_attention_mma
        fn.argtypes = [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int,
                       _c_int, _c_float, _c_int, _c_int, _c_void_p, _c_void_p]
        fn.restype = _c_int
        for name in ("ts_latent_attention_mma_rows", "ts_latent_attention_mma_keys"):
            getattr(lib, name).restype = _c_int
        fns = _latent_mma_libs[key] = (fn, lib.ts_latent_attention_mma_rows(), lib.ts_latent_attention_mma_keys())
    return fns


def latent_attention_splits(device: torch.device, num_seqs: int, rows_per_seq: int, plan_context: int, rank: int, rot_dim: int) -> int:
    """Into how many key ranges a step of few rows per sequence cuts each sequence's keys: the count
    that needs the fewest key blocks one after the other on an SM, given that one CTA is resident per
    SM: rounds of CTAs times (blocks per range + about a block and a half of fixed cost: the query
    rows, the first copy's latency, the partial sums).  A function of the batch's size and the
    planned context only (a captured step is replayed for every length)."""
    _, rows, keys = _latent_mma_fns(rank, rot_dim)
    ctas = max(1, num_seqs * -(-rows_per_seq // rows))
    blocks = max(1, -(-plan_context // keys))
    sms = _sm_count(device)
    best, best_cost = 1, None
    for splits in range(1, min(blocks, LATENT_MMA_MAX_SPLITS) + 1):
        cost = -(-ctas * splits // sms) * (-(-blocks // splits) + 1.5) + (0.5 if splits > 1 else 0.0)  # + the merge kernel
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = splits, cost
    return best


def latent_attention_mma(q_abs: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, gates: Optional[torch.Tensor],
                         cu_seqlens: torch.Tensor, context_lens: torch.Tensor, block_table: torch.Tensor, page_size: int, num_seqs: int,
                         max_seqlen_q: int, num_heads: int, rank: int, rot_dim: int, scale: float, window: int = 0, splits: int = 1) -> None:
    """Causal attention of absorbed queries over cached rows on the tensor cores (bfloat16): q_abs
    [T, H, rank+rot] holds exactly the tokens of sequences 0..num_seqs-1 (cu_seqlens), cache [pages,
    page, rank+rot], out [T, H, rank] = softmax(q . row * scale) @ row[:rank] * gates.  `splits` > 1
    cuts every sequence's keys into that many ranges (steps of few rows) merged by a second kernel."""
    flush_gemm_chain()
    _cuda_contig("q_abs", q_abs, torch.bfloat16)
    _cuda_contig("cache", cache, torch.bfloat16)
    _cuda_contig("out", out, torch.bfloat16)
    for name, t in (("cu_seqlens", cu_seqlens), ("context_lens", context_lens)):
        _cuda_contig(name, t, torch.int32)
    if block_table.dtype != torch.int32 or block_table.dim() != 2 or block_table.stride(1) != 1:
        raise KernelError("latent_attention_mma: block_table must be an int32 matrix with unit inner stride")
    T, H, D = q_abs.shape[0], num_heads, rank + rot_dim
    if not latent_attention_mma_supported(rank, rot_dim):
        raise KernelError(f"latent_attention_mma: rank {rank} and rotated width {rot_dim} must be multiples of 16 that fit shared memory")
    if q_abs.numel() != T * H * D or out.numel() != T * H * rank or tuple(cache.shape[-2:]) != (page_size, D):
        raise KernelError(f"latent_attention_mma: q_abs {tuple(q_abs.shape)}, out {tuple(out.shape)}, cache {tuple(cache.shape)} disagree")
    if cu_seqlens.numel() < num_seqs + 1 or context_lens.numel() < num_seqs or block_table.shape[0] < num_seqs:
        raise KernelError("latent_attention_mma: the index arrays are shorter than the batch")
    if gates is not None:
        _cuda_contig("gates", gates, torch.float32)
        if gates.numel() != T * H:
            raise KernelError("latent_attention_mma: gates must be [T, heads]")
    if not 1 <= splits <= LATENT_MMA_MAX_SPLITS:
        raise KernelError(f"latent_attention_mma: splits must lie in 1..{LATENT_MMA_MAX_SPLITS}")
    scratch = None
    if splits > 1:
        scratch = torch.empty(splits * T * H * (rank + 2), device=q_abs.device, dtype=torch.float32)
    fn, _, _ = _latent_mma_fns(rank, rot_dim)
    _check("latent_attention_mma", fn(
        q_abs.data_ptr(), cache.data_ptr(), out.data_ptr(), _ptr(gates), cu_seqlens.data_ptr(), context_lens.data_ptr(),
        block_table.data_ptr(), block_table.stride(0), page_size, num_seqs, max_seqlen_q, T, H, float(scale), int(window), int(splits),
        _ptr(scratch), _stream()))
    if splits > 1:
        global launch_count
        launch_count += 1  # the merge kernel


# ---------------------------------------------------------------------------
# tensor-core attention (one library per head size)

# Decode steps with 2..8 key splits: the splits of a (sequence, KV head) pair form a thread-block
# cluster and merge through its shared memory (TS_ATTENTION_CLUSTER=0: scratch and a second kernel).
ATTENTION_CLUSTER_MERGE = _os.environ.get("TS_ATTENTION_CLUSTER", "1") != "0"
# Decode steps fetch keys and values with the copy engine (TMA) where the sizes allow it: head sizes
# that are multiples of 64, pages of at least 8 slots that divide 64 or are multiples of it
# (TS_ATTENTION_TMA=0: 16-byte asynchronous copies by the threads, which take every size).
ATTENTION_DECODE_TMA = _os.environ.get("TS_ATTENTION_TMA", "1") != "0"
_attention_error: Optional[torch.Tensor] = None


def _pinned_word() -> torch.Tensor:
    """One zeroed int32 in pinned host memory that kernels may write and the host reads without a
    copy.  Made outside inference mode, so that the host may clear it from anywhere."""
    with torch.inference_mode(False):
        return torch.zeros(1, dtype=torch.int32).pin_memory()


def _word_is_set(word: torch.Tensor) -> bool:
    """Reads and clears an error word through its numpy view (plain memory, no tensor dispatch)."""
    view = word.numpy()
    if int(view[0]) == 0:
        return False
    view[0] = 0
    return True


def _attention_error_word() -> torch.Tensor:
    """One int in pinned host memory that the decode attention sets when a bounded wait gave up."""
    global _attention_error
    if _attention_error is None:
        _attention_error = _pinned_word()
    return _attention_error


ATTENTION_MMA_MAX_HEAD_DIM = 256
ATTENTION_MMA_MAX_SPLITS = 64
# TS_ATTENTION_MMA_DISTANCE=0 (for measurements): layers with a distance penalty run the CUDA-core kernel in bfloat16 too
ATTENTION_MMA_DISTANCE = _os.environ.get("TS_ATTENTION_MMA_DISTANCE", "1") != "0"
_attention_mma: dict[int, tuple] = {}


def attention_mma_supported(head_dim: int) -> bool:
    return head_dim % 16 == 0 and 16 <= head_dim <= ATTENTION_MMA_MAX_HEAD_DIM


def _attention_mma_fns(head_dim: int, scored: bool = False):
    """(run, scratch_floats) of the library built for `head_dim`; `scored`: the build that also knows a
    sink score per query head and a tanh cap on the scores (a library of its own, so that the kernels
    of models without either carry none of that code)."""
    key = (head_dim, True) if scored else head_dim
    fns = _attention_mma.get(key)
    if fns is None:
        if not attention_mma_supported(head_dim):
            raise KernelError(
                f"attention_paged_mma: head_dim must be a multiple of 16 between 16 and {ATTENTION_MMA_MAX_HEAD_DIM}, got {head_dim}")
        lib = _build.load_variant("attention_mma", {"TS_HEAD_DIM": head_dim, "TS_ATT_SCORED": 1} if scored else {"TS_HEAD_DIM": head_dim})
        run = lib.ts_attention_paged_mma_scored
        run.argtypes = ([_c_void_p] * 9 + [_c_int] * 7 + [_c_float, _c_int, _c_int, _c_int, _c_float, _c_float, _c_void_p, _c_int, _c_int,
                                                         _c_void_p, _c_void_p, _c_void_p, _c_void_p])
        run.restype = _c_int
        scratch = lib.ts_attention_mma_scratch_floats
        scratch.argtypes = [_c_ll, _c_int]
        scratch.restype = _c_ll
        if lib.ts_attention_mma_head_dim() != head_dim:
            raise KernelError("attention_paged_mma: the loaded library was built for another head size")
        lib.ts_attention_mma_set_cluster_merge.argtypes = [_c_int]
        lib.ts_attention_mma_set_cluster_merge(1 if ATTENTION_CLUSTER_MERGE else 0)
        lib.ts_attention_mma_set_decode_tma.argtypes = [_c_int]
        lib.ts_attention_mma_set_decode_tma(1 if ATTENTION_DECODE_TMA else 0)
        lib.ts_attention_mma_set_error_word.argtypes = [_c_void_p]
        lib.ts_attention_mma_set_error_word(_attention_error_word().data_ptr())
        lib.ts_attention_decode_flat.argtypes = [_c_void_p] * 9 + [_c_int] * 7 + [_c_float, _c_int, _c_int, _c_void_p]
        lib.ts_attention_decode_flat.restype = _c_int
        lib.ts_attention_decode_flat_ctas.restype = _c_int
        lib.ts_attention_decode_flat_scratch_floats.argtypes = [_c_int, _c_int]
        lib.ts_attention_decode_flat_scratch_floats.restype = _c_ll
        lib.ts_attention_mma_decode_slots.restype = _c_ll
        lib.ts_attention_mma_decode_rows.restype = _c_int
        lib.ts_attention_mma_last_launches.restype = _c_int
        if scored:
            _attention_scored[head_dim] = lib
        else:
            _attention_flat[head_dim] = lib
        fns = (run, scratch)
        _attention_mma[key] = fns
    return fns


_decode_slot_counts: dict[int, int] = {}


def _decode_slots(head_dim: int) -> int:
    """CTAs of the decode attention kernel that run at once on this device, as the library's
    occupancy query for the real kernel says."""
    n = _decode_slot_counts.get(head_dim)
    if n is None:
        _attention_mma_fns(head_dim)
        n = _decode_slot_counts[head_dim] = max(1, int(_attention_flat[head_dim].ts_attention_mma_decode_slots()))
    return n


def attention_decode_rows(head_dim: int) -> int:
    """The most query rows (tokens of the step x query heads per key/value head) of one sequence
    that the decode kernels take; steps with more go to the prompt kernels."""
    _attention_mma_fns(head_dim)
    return int(_attention_flat[head_dim].ts_attention_mma_decode_rows())


# The context length the split count of a decode step is planned for when the step may serve any
# length up to the model's (a captured graph does): long enough that a few thousand keys are spread
# over all SMs, short enough that a sequence of a few hundred keys is not cut into slivers
# (TS_DECODE_PLAN_CONTEXT overrides it for measurements).
ATTENTION_DECODE_PLAN_CONTEXT = int(_os.environ.get("TS_DECODE_PLAN_CONTEXT", "2048"))


def attention_decode_plan_context(max_context: int, window: int = 0) -> int:
    """The context length to plan a decode step's key splits for: the longest the step can meet,
    capped by the window (plus one key block) or by ATTENTION_DECODE_PLAN_CONTEXT."""
    cap = window + 64 if window > 0 else ATTENTION_DECODE_PLAN_CONTEXT
    return max(1, min(max_context, cap))


def attention_decode_splits(num_seqs: int, num_kv_heads: int, max_context: int, head_dim: int = 128) -> int:
    """How many CTAs share the keys of one sequence in a decode step.

    Each (sequence, KV head) pair is one unit of work that `splits` CTAs divide evenly.  The
    GPU runs `slots` CTAs at a time (shared memory allows a few per SM, fewer for large
    heads); the step takes ceil(pairs * splits / slots) waves, each as long as one CTA's
    share, so the count is chosen to fill whole waves: one wave for small batches, and for
    batches with more pairs than slots a count that makes the last wave nearly full.
    """
    slots = _decode_slots(head_dim)
    pairs = max(1, num_seqs * num_kv_heads)
    blocks = max(1, -(-max_context // 64))
    if _os.environ.get("TS_DECODE_SPLITS"):
        return max(1, min(int(_os.environ["TS_DECODE_SPLITS"]), blocks, ATTENTION_MMA_MAX_SPLITS))
    best, best_cost = 1, None
    for s in range(1, min(blocks, 16) + 1):
        waves = -(-pairs * s // slots)
        # per CTA: start and merge (about 3 us) + 2.5 us per 64-key block; merging the splits costs
        # little inside a thread-block cluster (up to 8 CTAs, all running at once), more through
        # scratch and a kernel of its own
        in_cluster = ATTENTION_CLUSTER_MERGE and s <= 8 and pairs * s <= slots
        merge = 0.0 if s == 1 else (0.8 if in_cluster else 1.5 + 0.15 * s)
        cost = waves * (3.0 + 2.5 * -(-blocks // s)) + merge
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


def attention_decode_plan(num_seqs: int, num_kv_heads: int, max_context: int, head_dim: int = 128) -> tuple[int, int]:
    """(splits, keys_per_split) for fixed-size key chunks: every (sequence, KV head) pair is cut
    into chunks of `keys_per_split` keys, one CTA each; `splits` chunks cover `max_context`, and
    sequences shorter than that use fewer of their CTAs.  For batches whose longest context is
    known when the step is launched."""
    pairs = max(1, num_seqs * num_kv_heads)
    chunk = 64 if pairs <= 16 else (128 if pairs <= 64 else 256)
    splits = -(-max(1, max_context) // chunk)
    while splits > ATTENTION_MMA_MAX_SPLITS:
        chunk *= 2
        splits = -(-max_context // chunk)
    if splits <= 1:
        return 1, 0
    return splits, chunk


def attention_paged_mma(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    out: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    context_lens: torch.Tensor,
    block_table: torch.Tensor,
    seq_index: torch.Tensor,
    page_size: int,
    num_seqs: int,
    max_seqlen_q: int,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    scale: float,
    window: int = 0,
    splits: int = 1,
    scratch: Optional[torch.Tensor] = None,
    keys_per_split: int = 0,
    fuse_merge: bool = True,
    chunk: int = 0,
    sink: Optional[float] = None,
    softcap: float = 0.0,
    head_sinks: Optional[torch.Tensor] = None,
    distance: Optional[tuple[torch.Tensor, torch.Tensor]] = None,
) -> None:
    """Causal attention over the paged cache on tensor cores (bfloat16).

    q/out [T,nq*d]; caches [pages,page,nkv,d]; cu_seqlens_q [B+1], context_lens [B],
    seq_index [T] i32; block_table [B,max_blocks] i32.  The tokens of a sequence are
    consecutive and end at context_lens[b] - 1.  splits > 1 spreads the keys of a
    sequence over several CTAs and needs `scratch` (float32, see attention_scratch_floats);
    keys_per_split > 0 (a multiple of 64) gives split s the keys [s * keys_per_split, ...),
    0 divides each sequence's keys evenly.  In decode steps the last CTA of each (sequence, KV
    head) pair merges the pair's splits itself (`fuse_merge`); otherwise a second kernel does.
    chunk > 0: a query sees only the keys of its own block of `chunk` positions (blocks count from
    position 0); sink: a score that joins every softmax's denominator without a value; head_sinks
    [nq] float32: one such score per query head; softcap > 0: the scaled score goes through
    softcap * tanh(s / softcap); distance = (r1, r2), [nq] float32 each: the scaled score of key j for the
    query at position i loses r1 * ln(1 + r2 * (i - j)).
    """
    flush_gemm_chain()
    if distance is not None:
        for name, t in zip(("distance r1", "distance r2"), distance):
            _cuda_contig(name, t, torch.float32)
            if t.numel() != num_heads:
                raise KernelError(f"attention: {name} must have one entry per query head ({num_heads}), got {t.numel()}")
    scored = head_sinks is not None or softcap > 0.0 or distance is not None
    run, _ = _attention_mma_fns(head_dim, scored)
    if head_sinks is not None:
        _cuda_contig("head_sinks", head_sinks, torch.float32)
        if head_sinks.numel() != num_heads or sink is not None:
            raise KernelError(f"attention: head_sinks must have one entry per query head ({num_heads}) and come without `sink`")
    for name, t in (("q", q), ("k_cache", k_cache), ("v_cache", v_cache), ("out", out)):
        _cuda_contig(name, t, torch.bfloat16)
    for name, t in (("cu_seqlens_q", cu_seqlens_q), ("context_lens", context_lens), ("block_table", block_table), ("seq_index", seq_index)):
        _cuda_contig(name, t, torch.int32)
    T = q.shape[0]
    nq, nkv, d = num_heads, num_kv_heads, head_dim
    if nq % nkv:
        raise KernelError(f"attention: {nq} query heads are no multiple of {nkv} key/value heads")
    if q.numel() != T * nq * d or out.numel() != T * nq * d:
        raise KernelError("attention: q/out do not match [T, heads*head_dim]")
    if tuple(k_cache.shape[-3:]) != (page_size, nkv, d) or k_cache.shape != v_cache.shape:
        raise KernelError(f"attention: caches must be [pages,{page_size},{nkv},{d}], got {tuple(k_cache.shape)} and {tuple(v_cache.shape)}")
    if block_table.dim() != 2 or block_table.shape[0] < num_seqs:
        raise KernelError("attention: block_table must be [B,max_blocks]")
    if cu_seqlens_q.numel() < num_seqs + 1 or context_lens.numel() < num_seqs or seq_index.numel() < T:
        raise KernelError("attention: cu_seqlens_q/context_lens/seq_index are shorter than the batch")
    if keys_per_split < 0 or keys_per_split % 64:
        raise KernelError(f"attention: keys_per_split must be a multiple of 64, got {keys_per_split}")
    if not (1 <= splits <= ATTENTION_MMA_MAX_SPLITS):
        raise KernelError(f"attention: splits must be 1..{ATTENTION_MMA_MAX_SPLITS}, got {splits}")
    if splits > 1:
        need = attention_scratch_floats(T * nq, splits, d)
        if scratch is None or scratch.dtype != torch.float32 or not scratch.is_cuda or scratch.numel() < need:
            raise KernelError(f"attention: splits={splits} needs {need} float32 of scratch")
    counters = None
    if fuse_merge and _FUSE_ATTENTION_MERGE and splits > 1 and max_seqlen_q * (nq // nkv) <= attention_decode_rows(d) and num_seqs * nkv <= _GEMM_MAX_TILES:
        counters = _attention_counters(q.device).data_ptr()
    _check("attention_paged_mma", run(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), _ptr(scratch),
        cu_seqlens_q.data_ptr(), context_lens.data_ptr(), block_table.data_ptr(), seq_index.data_ptr(),
        block_table.shape[1], page_size, T, num_seqs, max_seqlen_q, nq, nkv, float(scale), int(window), int(chunk),
        0 if sink is None else 1, 0.0 if sink is None else float(sink), float(softcap), _ptr(head_sinks), int(splits), int(keys_per_split),
        counters, _stream(), None if distance is None else distance[0].data_ptr(), None if distance is None else distance[1].data_ptr()))
    if splits > 1:
        global launch_count
        launch_count += (_attention_scored if scored else _attention_flat)[d].ts_attention_mma_last_launches() - 1  # the combine kernel, if one ran


# Decode steps whose (sequence, KV head) pairs times key splits do not all run at once go to the
# kernel that gives every CTA an even share of all key blocks instead (TS_ATTENTION_FLAT=0: never).
ATTENTION_DECODE_FLAT = _os.environ.get("TS_ATTENTION_FLAT", "1") != "0"
ATTENTION_FLAT_MAX_SEQS = 512
ATTENTION_FLAT_MAX_ROWS = 16
_attention_flat: dict[int, ctypes.CDLL] = {}
_attention_scored: dict[int, ctypes.CDLL] = {}  # the builds with per-head sinks and a score cap
_flat_ctas: dict[int, int] = {}


def attention_decode_flat_supported(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, num_seqs: int, max_seqlen_q: int) -> bool:
    """Whether the even-share decode kernel takes these sizes: head sizes that are multiples of 64,
    pages the copy engine can fetch (8 or more slots; 64 a multiple of the page or the page of 64),
    at most 16 rows (tokens x heads of a group) per sequence and KV head, at most 512 sequences."""
    return (head_dim % 64 == 0 and attention_mma_supported(head_dim) and num_kv_heads > 0 and num_heads % num_kv_heads == 0
            and page_size >= 8 and (64 % page_size == 0 or page_size % 64 == 0)
            and max_seqlen_q * (num_heads // num_kv_heads) <= ATTENTION_FLAT_MAX_ROWS and 0 < num_seqs <= ATTENTION_FLAT_MAX_SEQS
            and (num_kv_heads * head_dim * 2) % 16 == 0)


def attention_decode_prefers_flat(num_seqs: int, num_kv_heads: int, splits: int, head_dim: int) -> bool:
    """Whether a decode step of this many sequences is better served by the even-share kernel:
    when the CTAs of the split kernel would queue (measured at 8 KV heads of 128: equal at 32
    sequences, 19 % faster at 64, 10 % at 128; with fewer sequences the split kernel, whose
    splits merge inside a cluster, is faster)."""
    return ATTENTION_DECODE_FLAT and num_seqs * num_kv_heads * splits > _decode_slots(head_dim)


def attention_decode_flat_ctas(head_dim: int) -> int:
    """CTAs of the even-share decode kernel that the GPU runs at once: its grid."""
    n = _flat_ctas.get(head_dim)
    if n is None:
        _attention_mma_fns(head_dim)
        n = int(_attention_flat[head_dim].ts_attention_decode_flat_ctas())
        _flat_ctas[head_dim] = n
    return n


def attention_decode_flat(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    out: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    context_lens: torch.Tensor,
    block_table: torch.Tensor,
    seq_index: torch.Tensor,
    page_size: int,
    num_seqs: int,
    max_seqlen_q: int,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    scale: float,
    window: int = 0,
    ctas: int = 0,
) -> None:
    """Decode attention over the paged cache with an even share of key blocks per CTA (bfloat16).

    Arguments as attention_paged_mma.  The key blocks (64 keys) of all (sequence, KV head) pairs
    form one list that the CTAs of a fixed grid divide evenly on the device, whatever the lengths
    are; pairs that several CTAs share are merged by a second kernel.  `ctas` (0: as many as run
    at once) sets the grid."""
    flush_gemm_chain()
    _attention_mma_fns(head_dim)
    lib = _attention_flat[head_dim]
    for name, t in (("q", q), ("k_cache", k_cache), ("v_cache", v_cache), ("out", out)):
        _cuda_contig(name, t, torch.bfloat16)
    for name, t in (("cu_seqlens_q", cu_seqlens_q), ("context_lens", context_lens), ("block_table", block_table), ("seq_index", seq_index)):
        _cuda_contig(name, t, torch.int32)
    T = q.shape[0]
    nq, nkv, d = num_heads, num_kv_heads, head_dim
    if not attention_decode_flat_supported(nq, nkv, d, page_size, num_seqs, max_seqlen_q):
        raise KernelError(
            f"attention_decode_flat: takes head sizes that are multiples of 64, pages of 8 or more slots that divide 64 or are multiples of it, "
            f"at most {ATTENTION_FLAT_MAX_ROWS} rows per sequence and KV head and at most {ATTENTION_FLAT_MAX_SEQS} sequences; got "
            f"heads {nq}/{nkv} of {d}, page {page_size}, {num_seqs} sequences of up to {max_seqlen_q} tokens")
    if q.numel() != T * nq * d or out.numel() != T * nq * d:
        raise KernelError("attention_decode_flat: q/out do not match [T, heads*head_dim]")
    if tuple(k_cache.shape[-3:]) != (page_size, nkv, d) or k_cache.shape != v_cache.shape:
        raise KernelError(f"attention_decode_flat: caches must be [pages,{page_size},{nkv},{d}], got {tuple(k_cache.shape)} and {tuple(v_cache.shape)}")
    if block_table.dim() != 2 or block_table.shape[0] < num_seqs:
        raise KernelError("attention_decode_flat: block_table must be [B,max_blocks]")
    if cu_seqlens_q.numel() < num_seqs + 1 or context_lens.numel() < num_seqs or seq_index.numel() < T:
        raise KernelError("attention_decode_flat: cu_seqlens_q/context_lens/seq_index are shorter than the batch")
    most = attention_decode_flat_ctas(d)
    ctas = most if ctas <= 0 else min(int(ctas), most)
    scratch = torch.empty(int(lib.ts_attention_decode_flat_scratch_floats(num_seqs, ctas)), device=q.device, dtype=torch.float32)
    _check("attention_decode_flat", lib.ts_attention_decode_flat(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), scratch.data_ptr(),
        cu_seqlens_q.data_ptr(), context_lens.data_ptr(), block_table.data_ptr(), seq_index.data_ptr(),
        block_table.shape[1], page_size, T, num_seqs, max_seqlen_q, nq, nkv, float(scale), int(window), ctas, _stream()))
    global launch_count
    launch_count += 1  # the combine kernel


_FUSE_ATTENTION_MERGE = _os.environ.get("TS_FUSE_ATTENTION_MERGE", "0") != "0"  # measured: the separate merge kernel is a little faster
_attention_counter_tensors: dict[tuple[int, int], torch.Tensor] = {}


def _attention_counters(device: torch.device) -> torch.Tensor:
    """Per (device, stream): ticket counters of the decode attention's key splits (zero between launches)."""
    key = (device.index or 0, _stream())
    t = _attention_counter_tensors.get(key)
    if t is None:
        t = _attention_counter_tensors[key] = torch.zeros(_GEMM_MAX_TILES, dtype=torch.int32, device=device)
    return t


def attention_scratch_floats(rows: int, splits: int, head_dim: int) -> int:
    return rows * splits * (head_dim + 2) if splits > 1 else 0


# ---------------------------------------------------------------------------
# prompt attention on tcgen05 tensor cores (head size 128)

ATTENTION_TCGEN05_HEAD_DIM = 128
_attention_tcgen05 = None
_attention_tcgen05_scored = None  # the build with per-head sinks and a score cap
_USE_ATTENTION_TCGEN05 = _os.environ.get("TS_ATTENTION_TCGEN05", "1") != "0"


def _attention_tcgen05_fns(scored: bool = False):
    global _attention_tcgen05, _attention_tcgen05_scored
    if scored:
        if _attention_tcgen05_scored is None:
            _attention_tcgen05_fns()
            lib = _build.load_variant("attention_tcgen05", {"TS_HEAD_DIM": ATTENTION_TCGEN05_HEAD_DIM, "TS_ATT_SCORED": 1})
            run = lib.ts_attention_prefill_tcgen05_scored
            run.argtypes = _attention_tcgen05[0].argtypes
            run.restype = _c_int
            _attention_tcgen05_scored = (run, _attention_tcgen05[1])
        return _attention_tcgen05_scored
    if _attention_tcgen05 is None:
        lib = _build.load_variant("attention_tcgen05", {"TS_HEAD_DIM": ATTENTION_TCGEN05_HEAD_DIM})
        run = lib.ts_attention_prefill_tcgen05_scored
        run.argtypes = ([_c_void_p] * 7 + [_c_int, _c_int, _c_ll] + [_c_int] * 5 + [_c_float, _c_int, _c_int, _c_int, _c_float, _c_float, _c_void_p,
                                                                                     _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p])
        run.restype = _c_int
        ok = lib.ts_attention_tcgen05_supported
        ok.argtypes = [_c_int, _c_int, _c_int]
        ok.restype = _c_int
        _attention_tcgen05 = (run, ok)
    return _attention_tcgen05


def attention_tcgen05_supported(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 prompt-attention kernel takes these sizes: head size 128, at most 128
    query heads per key/value head (a tile of 128 rows holds whole tokens: 128 // group of them), a
    page size of at least 8 that divides 64 or is a multiple of 128."""
    if not _USE_ATTENTION_TCGEN05 or head_dim != ATTENTION_TCGEN05_HEAD_DIM:
        return False
    if num_kv_heads <= 0 or num_heads % num_kv_heads or num_heads // num_kv_heads > 128:
        return False
    return page_size >= 8 and (64 % page_size == 0 or page_size % 128 == 0)


def attention_prefill_tcgen05(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    out: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    context_lens: torch.Tensor,
    block_table: torch.Tensor,
    page_size: int,
    num_seqs: int,
    max_seqlen_q: int,
    num_heads: int,
    num_kv_heads: int,
    scale: float,
    window: int = 0,
    mode: int = 0,
    chunk: int = 0,
    sink: Optional[float] = None,
    softcap: float = 0.0,
    head_sinks: Optional[torch.Tensor] = None,
    distance: Optional[tuple[torch.Tensor, torch.Tensor]] = None,
) -> None:
    """Causal attention of prompt portions over the paged cache, tcgen05 tensor cores, head size 128.

    Same arguments and meaning as attention_paged_mma (without seq_index, which it does not need).
    `mode`: 1 one tile of 128 rows per CTA, 2 two tiles per CTA with the roles in warps of
    their own, 0 chooses by the longest portion.
    """
    flush_gemm_chain()
    run, ok = _attention_tcgen05_fns(head_sinks is not None or softcap > 0.0 or distance is not None)
    d = ATTENTION_TCGEN05_HEAD_DIM
    if distance is not None:
        for name, t in zip(("distance r1", "distance r2"), distance):
            _cuda_contig(name, t, torch.float32)
            if t.numel() != num_heads:
                raise KernelError(f"attention_prefill_tcgen05: {name} must have one entry per query head ({num_heads}), got {t.numel()}")
    for name, t in (("q", q), ("k_cache", k_cache), ("v_cache", v_cache), ("out", out)):
        _cuda_contig(name, t, torch.bfloat16)
    for name, t in (("cu_seqlens_q", cu_seqlens_q), ("context_lens", context_lens), ("block_table", block_table)):
        _cuda_contig(name, t, torch.int32)
    T = q.shape[0]
    nq, nkv = num_heads, num_kv_heads
    if not ok(nq, nkv, page_size):
        raise KernelError(
            f"attention_prefill_tcgen05: needs at most 128 query heads per key/value head and a page size of at least 8 that divides 64 or is a multiple of 128; "
            f"got {nq} query heads, {nkv} key/value heads, pages of {page_size}")
    if q.numel() != T * nq * d or out.numel() != T * nq * d:
        raise KernelError("attention_prefill_tcgen05: q/out do not match [T, heads*128]")
    if tuple(k_cache.shape[-3:]) != (page_size, nkv, d) or k_cache.shape != v_cache.shape:
        raise KernelError(f"attention_prefill_tcgen05: caches must be [pages,{page_size},{nkv},{d}], got {tuple(k_cache.shape)} and {tuple(v_cache.shape)}")
    if block_table.dim() != 2 or block_table.shape[0] < num_seqs:
        raise KernelError("attention_prefill_tcgen05: block_table must be [B,max_blocks]")
    if cu_seqlens_q.numel() < num_seqs + 1 or context_lens.numel() < num_seqs:
        raise KernelError("attention_prefill_tcgen05: cu_seqlens_q/context_lens are shorter than the batch")
    if head_sinks is not None:
        _cuda_contig("head_sinks", head_sinks, torch.float32)
        if head_sinks.numel() != nq or sink is not None:
            raise KernelError(f"attention_prefill_tcgen05: head_sinks must have one entry per query head ({nq}) and come without `sink`")
    _, error = _gemm_workspace(q.device)
    _check("attention_prefill_tcgen05", run(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
        cu_seqlens_q.data_ptr(), context_lens.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], page_size, k_cache.shape[0] * page_size, T, num_seqs, max_seqlen_q, nq, nkv,
        float(scale), int(window), int(chunk), 0 if sink is None else 1, 0.0 if sink is None else float(sink), float(softcap),
        _ptr(head_sinks), int(mode), error.data_ptr(), _stream(), None if distance is None else distance[0].data_ptr(),
        None if distance is None else distance[1].data_ptr()))


# ---------------------------------------------------------------------------
# skinny GEMM on tcgen05 tensor cores (decode steps)

GEMM_SKINNY_MAX_ROWS = 128
_SIGNATURES["ts_gemm_skinny_bf16"] = [
    _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_ll, _c_ll, _c_ll, _c_int,
    _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_ll, _c_void_p,
]
# How much of the next GEMM's weights a GEMM asks into L2 while its own last tiles are finished.
# Measured on the decode step at batch 8 (ms per step, the weights themselves passing through the
# L2 as "evict first"): none 3.87, 8 MB 3.83, 16 MB 3.80, 24 MB 3.82, 32 MB 3.84, 48 MB 3.86,
# 96 MB 3.94 (the requests then compete with the kernel's own tail).  TS_GEMM_PREFETCH_MB
# overrides it for measurements.
GEMM_PREFETCH_BYTES = int(_os.environ.get("TS_GEMM_PREFETCH_MB", "16")) << 20
_gemm_workspaces: dict[tuple[int, int], tuple[torch.Tensor, torch.Tensor]] = {}
_CHAIN_SYNC_WORDS = 512  # at least ts_gemm_chain_sync_words(), on a 128-byte boundary behind the tickets


def _gemm_workspace(device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    """Per (device, stream): the ticket counters of the K-split tiles (zero between launches)
    and the error word, which lives in pinned host memory so the host can look at it without
    a copy."""
    key = (device.index or 0, _stream())
    ws = _gemm_workspaces.get(key)
    if ws is None:
        counters = torch.zeros(_GEMM_MAX_TILES + _CHAIN_SYNC_WORDS, dtype=torch.int32, device=device)  # tickets, then the chain's barrier words
        error = _pinned_word()
        ws = _gemm_workspaces[key] = (counters, error)
    return ws


_gemm_partials: dict[tuple[int, int], torch.Tensor] = {}
_gemm_partials_outgrown: list[torch.Tensor] = []
_gemm_scratch_need: dict[tuple[int, int, int], int] = {}


def _gemm_partial(device: torch.device, M: int, N: int, K: int) -> torch.Tensor:
    """Per (device, stream): the float32 scratch in which CTAs that share a tile meet.  One buffer
    serves every launch on the stream (it only grows): a GEMM stores nothing before the kernels
    ahead of it are done, so two launches never use it at once."""
    need = _gemm_scratch_need.get((M, N, K))
    if need is None:
        scratch_floats = library().ts_gemm_skinny_scratch_floats
        scratch_floats.restype = _c_ll
        need = _gemm_scratch_need[(M, N, K)] = max(4, int(scratch_floats(M, N, K)))
    key = (device.index or 0, _stream())
    buf = _gemm_partials.get(key)
    if buf is None or buf.numel() < need:
        if buf is not None:
            _gemm_partials_outgrown.append(buf)  # a captured graph may still name it: never handed back
        buf = _gemm_partials[key] = torch.empty(max(need, 1 << 20), dtype=torch.float32, device=device)
    return buf


class _MatrixFacts:
    """What the GEMM wrappers ask of a weight matrix again and again, looked up once and kept on the
    tensor object (a weight does not change its place or shape while it lives)."""

    __slots__ = ("ok", "ptr", "rows", "cols", "ld", "nbytes")

    def __init__(self, w: torch.Tensor) -> None:
        self.ptr = w.data_ptr()
        self.rows, self.cols = (int(w.shape[0]), int(w.shape[1])) if w.dim() == 2 else (0, 0)
        self.ld = int(w.stride(0)) if w.dim() == 2 else 0
        self.nbytes = w.numel() * w.element_size()
        self.ok = bool(
            w.dim() == 2 and w.is_cuda and w.dtype == torch.bfloat16 and self.cols % 8 == 0 and w.stride(1) == 1
            and self.ld % 8 == 0 and self.ptr % 16 == 0 and -(-self.rows // 128) <= _GEMM_MAX_TILES)


def _facts(w: torch.Tensor) -> _MatrixFacts:
    f = getattr(w, "_ts_facts", None)
    if f is None or f.ptr != w.data_ptr():
        f = _MatrixFacts(w)
        try:
            w._ts_facts = f
        except (AttributeError, RuntimeError):  # an object that takes no attributes: look it up every time
            pass
    return f


def matrix_streams_through_own_gemm(w: Optional[torch.Tensor]) -> bool:
    """Whether `w` ([out, in], bfloat16, on the device, rows on 16-byte boundaries, in % 8 == 0) is a
    weight the engine's own few-row GEMM takes."""
    return w is not None and _facts(w).ok


def gemm_skinny_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    M, K = x.shape
    return (
        _facts(w).ok and x.dtype == torch.bfloat16 and 0 < M <= GEMM_SKINNY_MAX_ROWS and K % 8 == 0
        and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
    )


_gemm_scratch_ptrs: dict[tuple[int, int], tuple[int, int, int, int]] = {}


def _gemm_scratch(device: torch.device, M: int, N: int, K: int) -> tuple[int, int, int, int]:
    """(partial sums, ticket counters, error word, stream) as plain addresses for one launch on the
    current stream: the buffers of _gemm_partial and _gemm_workspace, looked up with one query of
    the stream."""
    stream = _stream()
    key = (device.index or 0, stream)
    need = _gemm_scratch_need.get((M, N, K))
    got = _gemm_scratch_ptrs.get(key)
    if need is None or got is None or got[3] < need:
        partial = _gemm_partial(device, M, N, K)
        counters, error = _gemm_workspace(device)
        got = _gemm_scratch_ptrs[key] = (partial.data_ptr(), counters.data_ptr(), error.data_ptr(), partial.numel())
    return got[0], got[1], got[2], stream


def gemm_skinny_bf16(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, prefetch: Optional[torch.Tensor] = None) -> None:
    """out[M,N] = x[M,K] @ w[N,K]^T for M <= 128 on the tcgen05 tensor cores.

    x, w bfloat16 with unit inner stride and rows that start on 16-byte boundaries; out
    bfloat16 or float32.  The work is spread evenly over all SMs; tiles that two CTAs share
    meet in a float32 scratch that this wrapper allocates.  `prefetch`: the weights the next
    product will read; the kernel asks for their start to be brought into L2 while it finishes.
    """
    if not (x.is_cuda and w.is_cuda and out.is_cuda):
        raise KernelError("gemm_skinny_bf16: CUDA tensors only (there is no CPU path)")
    if not gemm_skinny_supported(x, w):
        raise KernelError(
            f"gemm_skinny_bf16: needs bfloat16, at most {GEMM_SKINNY_MAX_ROWS} rows, K a multiple of 8 and 16-byte "
            f"aligned rows; got x {tuple(x.shape)} {x.dtype} strides {x.stride()}, w {tuple(w.shape)} {w.dtype}")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N) or out.stride(1) != 1 or out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"gemm_skinny_bf16: shapes disagree: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} {out.dtype}")
    partial, counters, error, stream = _gemm_scratch(x.device, M, N, K)
    pf = None if prefetch is None else _facts(prefetch)
    _check_product("gemm_skinny_bf16", _fn("ts_gemm_skinny_bf16")(
        x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, x.stride(0), w.stride(0), out.stride(0),
        1 if out.dtype == torch.float32 else 0, partial, counters, error,
        None if pf is None else pf.ptr, 0 if pf is None else min(pf.nbytes, GEMM_PREFETCH_BYTES),
        stream), x, w, out)


_SIGNATURES["ts_gemm_skinny_fused"] = [
    _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_ll, _c_ll, _c_ll, _c_int,
    _c_int, _c_void_p, _c_int, _c_float, _c_float, _c_void_p, _c_ll, _c_void_p, _c_void_p, _c_void_p,
    _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_ll, _c_void_p,
]
GEMM_FUSED_MAX_ROWS = 32
GEMM_EPILOGUE_PLAIN, GEMM_EPILOGUE_SWIGLU, GEMM_EPILOGUE_RESIDUAL_NORM = 0, 1, 2


def gemm_skinny_fused(
    x: torch.Tensor,
    w: torch.Tensor,
    *,
    out: Optional[torch.Tensor] = None,
    mode: int = GEMM_EPILOGUE_PLAIN,
    scale_ssq: Optional[torch.Tensor] = None,
    scale_width: int = 1,
    scale_eps: float = 0.0,
    hidden: Optional[torch.Tensor] = None,
    norm_weight: Optional[torch.Tensor] = None,
    xprime: Optional[torch.Tensor] = None,
    ssq_out: Optional[torch.Tensor] = None,
    prefetch: Optional[torch.Tensor] = None,
) -> None:
    """x[M,K] @ w[N,K]^T on the tcgen05 tensor cores (M <= 32) with the work of the neighbouring
    small kernels done where each tile is finished.

    scale_ssq [tiles, M] float32: x lacks its norm's 1/rms (x = source * norm weight); the sums
    of squares of the source rows per 128 columns, as a GEMM in mode 2 leaves them; every row m of
    the product is multiplied by rsqrt(sum_m / scale_width + scale_eps).
    mode GEMM_EPILOGUE_PLAIN: out[M,N] bf16 or float32.
    mode GEMM_EPILOGUE_SWIGLU: the rows of w come in blocks of 128, 64 gate rows and then the 64 up
      rows of the same outputs; out[M,N/2] bf16 = silu(gate) * up.
    mode GEMM_EPILOGUE_RESIDUAL_NORM: hidden[M,N] float32 += product; xprime[M,N] bf16 = hidden *
      norm_weight; ssq_out[ceil(N/128), M] float32 = sums of squares of the new hidden rows.
    """
    if not gemm_skinny_supported(x, w) or x.shape[0] > GEMM_FUSED_MAX_ROWS:
        raise KernelError(
            f"gemm_skinny_fused: needs bfloat16, at most {GEMM_FUSED_MAX_ROWS} rows, K a multiple of 8 and 16-byte "
            f"aligned rows; got x {tuple(x.shape)} {x.dtype} strides {x.stride()}, w {tuple(w.shape)} {w.dtype}")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm_skinny_fused: shapes disagree: x {tuple(x.shape)}, w {tuple(w.shape)}")
    ldo, out_f32 = 0, 0
    if mode in (GEMM_EPILOGUE_PLAIN, GEMM_EPILOGUE_SWIGLU):
        cols = N if mode == GEMM_EPILOGUE_PLAIN else N // 2
        if out is None or not out.is_cuda or tuple(out.shape) != (M, cols) or out.stride(1) != 1:
            raise KernelError(f"gemm_skinny_fused: out must be [{M},{cols}]")
        if out.dtype not in ((torch.bfloat16, torch.float32) if mode == GEMM_EPILOGUE_PLAIN else (torch.bfloat16,)):
            raise KernelError(f"gemm_skinny_fused: out dtype {out.dtype} not taken in mode {mode}")
        if mode == GEMM_EPILOGUE_SWIGLU and N % 128:
            raise KernelError("gemm_skinny_fused: the gate/up blocks need N to be a multiple of 128")
        ldo, out_f32 = out.stride(0), 1 if out.dtype == torch.float32 else 0
    elif mode == GEMM_EPILOGUE_RESIDUAL_NORM:
        tiles = -(-N // 128)
        ok = (
            hidden is not None and hidden.dtype == torch.float32 and tuple(hidden.shape) == (M, N) and hidden.is_contiguous()
            and xprime is not None and xprime.dtype == torch.bfloat16 and tuple(xprime.shape) == (M, N) and xprime.is_contiguous()
            and norm_weight is not None and norm_weight.dtype == torch.float32 and norm_weight.numel() == N and norm_weight.is_contiguous()
            and ssq_out is not None and ssq_out.dtype == torch.float32 and ssq_out.numel() >= tiles * M and ssq_out.is_contiguous()
        )
        if not ok:
            raise KernelError("gemm_skinny_fused: mode 2 needs hidden f32 [M,N], xprime bf16 [M,N], norm_weight f32 [N], ssq_out f32 [tiles,M]")
    else:
        raise KernelError(f"gemm_skinny_fused: no mode {mode}")
    scale_tiles = 0
    if scale_ssq is not None:
        if scale_ssq.dtype != torch.float32 or not scale_ssq.is_contiguous() or scale_ssq.dim() != 2 or scale_ssq.shape[1] != M:
            raise KernelError("gemm_skinny_fused: scale_ssq must be float32 [tiles, M]")
        scale_tiles = scale_ssq.shape[0]
    partial, counters, error, stream = _gemm_scratch(x.device, M, N, K)
    pf = None if prefetch is None else _facts(prefetch)
    _check_product("gemm_skinny_fused", _fn("ts_gemm_skinny_fused")(
        x.data_ptr(), w.data_ptr(), _ptr(out), M, N, K, x.stride(0), w.stride(0), ldo, out_f32,
        int(mode), _ptr(scale_ssq), scale_tiles, float(scale_width), float(scale_eps),
        _ptr(hidden), N, _ptr(norm_weight), _ptr(xprime), _ptr(ssq_out),
        partial, counters, error,
        None if pf is None else pf.ptr, 0 if pf is None else min(pf.nbytes, GEMM_PREFETCH_BYTES),
        stream), x, w, out, scale_ssq, hidden, norm_weight, xprime, ssq_out)


_SIGNATURES["ts_gemm_skinny_qk_rope"] = [
    _c_void_p, _c_void_p, _c_int, _c_int, _c_ll, _c_ll, _c_int, _c_int,
    _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
    _c_void_p, _c_void_p, _c_float, _c_void_p, _c_void_p,
    _c_void_p, _c_int, _c_float, _c_float,
    _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_ll, _c_void_p,
]
GEMM_QK_ROPE_HEAD_DIM = 128

_SIGNATURES["ts_rope_cos_sin"] = [_c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p]


def rope_cos_sin(positions: torch.Tensor, inv_freq: torch.Tensor, num_tokens: int) -> torch.Tensor:
    """[num_tokens, len(inv_freq), 2] float32: (cos, sin) of positions[t] * inv_freq[j], the float32
    product and functions that the rotating kernels use themselves.  A step computes it once for
    all layers that rotate with the same frequencies."""
    _cuda_contig("positions", positions, torch.int32)
    _cuda_contig("inv_freq", inv_freq, torch.float32)
    if positions.numel() < num_tokens:
        raise KernelError("rope_cos_sin: positions are shorter than the tokens")
    half = inv_freq.numel()
    out = torch.empty((num_tokens, half, 2), device=positions.device, dtype=torch.float32)
    _check("rope_cos_sin", _fn("ts_rope_cos_sin")(positions.data_ptr(), inv_freq.data_ptr(), num_tokens, half, out.data_ptr(), _stream()))
    return out


def gemm_qk_rope_store(
    x: torch.Tensor,
    w: torch.Tensor,
    q_out: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    slot_mapping: torch.Tensor,
    positions: torch.Tensor,
    q_norm_weight: Optional[torch.Tensor],
    k_norm_weight: Optional[torch.Tensor],
    eps: float,
    inv_freq: Optional[torch.Tensor],
    num_heads: int,
    num_kv_heads: int,
    *,
    scale_ssq: Optional[torch.Tensor] = None,
    scale_width: int = 1,
    scale_eps: float = 0.0,
    prefetch: Optional[torch.Tensor] = None,
    cos_sin: Optional[torch.Tensor] = None,
) -> None:
    """The q/k/v projection (w [(nq + 2 nkv) * 128, K], heads of 128) with qk_norm_rope_store's work
    done in the product's epilogue: per-head RMS norm of q and k, rotate-half rotation over the
    whole head (inv_freq [64]) or none, q to q_out [M, nq * 128], k and v to their cache slots.
    At most 32 rows.  scale_ssq as in gemm_skinny_fused.  cos_sin: rope_cos_sin(positions, inv_freq,
    M) if the caller has it (the epilogue then reads the angles' cosines and sines instead of
    computing them)."""
    nq, nkv, d = num_heads, num_kv_heads, GEMM_QK_ROPE_HEAD_DIM
    if not gemm_skinny_supported(x, w) or x.shape[0] > GEMM_FUSED_MAX_ROWS:
        raise KernelError(f"gemm_qk_rope_store: needs bfloat16, at most {GEMM_FUSED_MAX_ROWS} rows and 16-byte aligned rows")
    M, K = x.shape
    if tuple(w.shape) != ((nq + 2 * nkv) * d, K):
        raise KernelError(f"gemm_qk_rope_store: w must be [{(nq + 2 * nkv) * d},{K}], got {tuple(w.shape)}")
    _cuda_contig("q_out", q_out, torch.bfloat16)
    _cuda_contig("k_cache", k_cache, torch.bfloat16)
    _cuda_contig("v_cache", v_cache, torch.bfloat16)
    _cuda_contig("slot_mapping", slot_mapping, torch.int32)
    _cuda_contig("positions", positions, torch.int32)
    if q_out.numel() != M * nq * d or tuple(k_cache.shape[-2:]) != (nkv, d) or k_cache.shape != v_cache.shape:
        raise KernelError("gemm_qk_rope_store: q_out must hold [M, nq*128], the caches [.., nkv, 128]")
    if slot_mapping.numel() < M or positions.numel() < M:
        raise KernelError("gemm_qk_rope_store: slot_mapping/positions are shorter than the rows")
    for name, t, n in (("q_norm_weight", q_norm_weight, d), ("k_norm_weight", k_norm_weight, d), ("inv_freq", inv_freq, d // 2)):
        if t is not None and (t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous() or t.numel() != n):
            raise KernelError(f"gemm_qk_rope_store: {name} must be {n} float32 on the device")
    scale_tiles = 0
    if scale_ssq is not None:
        if scale_ssq.dtype != torch.float32 or not scale_ssq.is_contiguous() or scale_ssq.dim() != 2 or scale_ssq.shape[1] != M:
            raise KernelError("gemm_qk_rope_store: scale_ssq must be float32 [tiles, M]")
        scale_tiles = scale_ssq.shape[0]
    if cos_sin is not None and (inv_freq is None or cos_sin.dtype != torch.float32 or not cos_sin.is_cuda or not cos_sin.is_contiguous()
                                or cos_sin.numel() < M * d):
        raise KernelError(f"gemm_qk_rope_store: cos_sin must be float32 [M, {d // 2}, 2] on the device, beside inv_freq")
    partial, counters, error, stream = _gemm_scratch(x.device, M, w.shape[0], K)
    pf = None if prefetch is None else _facts(prefetch)
    _check_product("gemm_qk_rope_store", _fn("ts_gemm_skinny_qk_rope")(
        x.data_ptr(), w.data_ptr(), M, K, x.stride(0), w.stride(0), nq, nkv,
        q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), slot_mapping.data_ptr(), positions.data_ptr(),
        _ptr(q_norm_weight), _ptr(k_norm_weight), float(eps), _ptr(inv_freq), _ptr(cos_sin),
        _ptr(scale_ssq), scale_tiles, float(scale_width), float(scale_eps),
        partial, counters, error,
        None if pf is None else pf.ptr, 0 if pf is None else min(pf.nbytes, GEMM_PREFETCH_BYTES),
        stream), x, w, q_out, k_cache, v_cache, slot_mapping, positions, q_norm_weight, k_norm_weight, inv_freq, cos_sin, scale_ssq)


_SIGNATURES["ts_wait_gives_up_probe"] = [_c_void_p, _c_int, _c_void_p]


def wait_gives_up_probe(device: torch.device, limit: int = 4096) -> None:
    """Launches a kernel whose only bounded wait runs out (an mbarrier nothing feeds, `limit`
    tries) and which then raises the current stream's error word exactly as the tcgen05 kernels
    do: the way to see the error path work without a fault.  check_device_errors() raises after
    the next synchronisation."""
    flush_gemm_chain()
    _, error = _gemm_workspace(device)
    _check("wait_gives_up_probe", _fn("ts_wait_gives_up_probe")(error.data_ptr(), int(limit), _stream()))


def library_mm(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None, float32_out: bool = False) -> torch.Tensor:
    """x [T, in] @ weight[out, in]^T by the library GEMM (cuBLAS through torch.mm), for steps of more
    rows than the engine's own weight-streaming kernel takes; a float32 result keeps the sums
    unrounded (the logits)."""
    flush_gemm_chain()  # the library reads x by itself
    if float32_out:
        return torch.mm(x, weight.t(), out_dtype=torch.float32)
    return torch.mm(x, weight.t(), out=out)


# Timers per kernel class, for eager steps (a replayed graph has no calls to time): switched on,
# every launching function of this module is wrapped so that a pair of CUDA events brackets what it
# launches; switched off, the functions are the plain ones again and nothing is paid.
_TIMED = ("embed_gather", "feed_tokens", "add_rmsnorm", "residual_add", "swiglu", "qk_norm_rope_store", "attention_paged_simple",
          "sample", "sgemm_nt", "attention_paged_mma", "attention_decode_flat", "attention_prefill_tcgen05", "gemm_skinny_bf16",
          "gemm_skinny_fused", "rope_cos_sin", "gemm_qk_rope_store", "library_mm", "sgemm_nt_batched", "library_bmm", "pair_hash_embed",
          "rmsnorm_add", "round_rows", "latent_prepare", "latent_attention_simple", "latent_attention_mma", "gelu_tanh", "capped_glu", "gelu_gate_rows",
          "router_topk", "router", "moe_plan", "moe_gate_up", "moe_down", "moe_combine", "branch_norm_add", "stream_add",
          "qk_joint_norm_rope_store", "gla_scan", "gla_norm_gate", "linear_scan", "rows_dot_f32", "mlstm_gate_scan", "mlstm_norm_gate",
          "ssm_conv", "ssm_gate_norm", "scale_rows", "weighted_sum", "rope_table", "qkv_prepare", "gate_rows", "causal_conv", "delta_scan",
          "softcap_rows")
_plain_functions: dict[str, object] = {}
_kernel_events: list[tuple[str, "torch.cuda.Event", "torch.cuda.Event"]] = []


def time_kernels(on: bool) -> None:
    """Switches the per-class timers on or off (see kernel_times)."""
    import functools

    g = globals()
    if on and not _plain_functions:
        for name in _TIMED:
            plain = g[name]

            def timed(*args, _plain=plain, _name=name, **kwargs):
                if torch.cuda.is_current_stream_capturing():
                    return _plain(*args, **kwargs)
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                result = _plain(*args, **kwargs)
                stop.record()
                _kernel_events.append((_name, start, stop))
                return result

            _plain_functions[name] = plain
            g[name] = functools.wraps(plain)(timed)
    elif not on and _plain_functions:
        for name, plain in _plain_functions.items():
            g[name] = plain
        _plain_functions.clear()


def kernel_times() -> dict[str, dict]:
    """{function: {"calls": n, "ms": device time between the events around its launches}} since the
    last call, after waiting for the device.  Classes: the function names of this module
    (`gemm_skinny_fused` includes the norms and activations folded into it; `library_mm` is cuBLAS)."""
    torch.cuda.synchronize()
    out: dict[str, dict] = {}
    for name, start, stop in _kernel_events:
        row = out.setdefault(name, {"calls": 0, "ms": 0.0})
        row["calls"] += 1
        row["ms"] += start.elapsed_time(stop)
    _kernel_events.clear()
    for row in out.values():
        row["ms"] = round(row["ms"], 3)
    return out


def check_device_errors() -> None:
    """Raises if a kernel reported that one of its bounded waits gave up.  Cheap: reads
    pinned host words; call it wherever the host has just synchronised anyway."""
    if _attention_error is not None and _word_is_set(_attention_error):
        raise KernelError("decode attention: a wait on an mbarrier gave up (the kernel returned early)")
    for (dev, _), (_, error) in _gemm_workspaces.items():
        if _word_is_set(error):
            raise KernelError(f"a tcgen05 kernel on cuda:{dev} (skinny GEMM or prompt attention): a wait on an mbarrier gave up (the kernel returned early)")
