"""Two designs side by side at equal size: Fegetar (latent attention, dense and routed feed-forwards)
and Qwen3 dense (grouped-query attention, SwiGLU), random weights, a few layers of widths that
resemble a real model's.  For each: one prompt of PREFILL_TOKENS tokens as one step, decode steps
at two batch sizes (graphs, as generation runs them), and the device time per kernel class of an
eager prompt step and an eager decode step, with the attention kernels' distance from their
rooflines (prompt: flops against the measured bf16 peak; decode: cache bytes against the measured
copy bandwidth).  `python bench.py --designs` prints one JSON line.

`python bench.py --designs dazilix` does the same for Dazilix (attention inside blocks of positions
with a sink, gated linear attention, routed SwiGLU experts, every sublayer between two norms)
beside Qwen3 dense at equal width, depth, heads and feed-forward weight per token, and adds the
recurrent mixer's and the norm kernels' distance from their rooflines.

`python bench.py --designs pekunex` runs Pekunex (attention with a score cap, a gate and biases;
attention with a sink per head beside a matrix memory; a state-space layer; dense SwiGLU) beside
Dazilix, the closest design the engine has (attention with a sink and a linear recurrence), at equal
width, depth, heads and feed-forward weight per token, with the distance of Pekunex's attention,
recurrence and small kernels from their rooflines next to the like kernels of Dazilix.

`python bench.py --designs vasosun` runs Vasosun (windowed attention with a query temperature and a
distance penalty, latent attention with a query latent and a layer that reads its cached rows, the
gated delta rule, routed experts without gates among which identity experts, every sublayer between
two norms and behind a short convolution of its input) beside Dazilix, the closest design the engine
has (the same block arrangement, attention and a linear recurrence, routed experts), at equal width,
depth, heads and expert sizes, with the distance of Vasosun's attention, recurrence and small kernels
from their rooflines next to the like kernels of Dazilix.
"""

from __future__ import annotations

from typing import Any

PREFILL_TOKENS = 2048
DECODE_CONTEXT = 1024
DECODE_BATCHES = (8, 64)
PAGE = 16
VOCAB = 32768

# name -> (width, heads, layers); the latent is 512 + 64 wide and a head 128 (+ 64 rotated) as in
# published models of this kind; half of the layers are dense, half routed
SIZES = {
    "w2048": dict(width=2048, heads=16, layers=4, dense_ff=8192, experts=16, top=2, expert_ff=1024, shared_ff=2048),
    "w4096": dict(width=4096, heads=32, layers=4, dense_ff=12288, experts=32, top=4, expert_ff=1536, shared_ff=3072),
}


def fegetar_config(s: dict) -> dict:
    mixer = {"heads": s["heads"], "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "scale": 192 ** -0.5,
             "rot": {"base": 1000000.0, "dims": 64}}
    dense = {"kind": "dense", "ff": s["dense_ff"]}
    moe = {"kind": "moe", "router": {"experts": s["experts"], "top": s["top"]}, "expert": {"ff": s["expert_ff"], "limit": 7.0},
           "shared": {"ff": s["shared_ff"], "limit": 7.0}}
    return {"architecture": "Fegetar", "vocab": VOCAB, "width": s["width"], "norm": {"eps": 1e-5},
            "embedding": {"bigram": {"buckets": 65521, "mul_prev": 1000003, "mul_cur": 31}}, "token_side": {"dim": 64},
            "layers": [{"type": "latent_attention", "mixer": mixer, "mlp": dense if i % 2 == 0 else moe} for i in range(s["layers"])]}


def fegetar_ff_params(s: dict) -> float:
    """Feed-forward weights a token reads per layer, averaged over the dense and the routed layers."""
    W = s["width"]
    return (2 * W * s["dense_ff"] + 3 * W * (s["top"] * s["expert_ff"] + s["shared_ff"])) / 2


def qwen3_config(s: dict) -> dict:
    W = s["width"]
    inter = int(round(fegetar_ff_params(s) / (3 * W) / 64)) * 64  # SwiGLU of the same weight per token
    return {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": s["layers"], "hidden_size": W,
            "num_attention_heads": s["heads"], "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": inter, "vocab_size": VOCAB,
            "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 8192,
            "hidden_act": "silu", "attention_bias": False, "torch_dtype": "bfloat16"}


# Dazilix at the same widths: three attention layers and one recurrent layer, heads of 128, blocks of
# positions long enough to hold the prompt (so that its attention does the work of the dense model's),
# routed experts in every layer; the recurrent layer's state is [heads, 64, 128] float32 per request.
DAZILIX_SIZES = {
    "w2048": dict(width=2048, heads=16, layers=4, experts=16, top=2, expert_ff=1024, gla_dim=64, gla_vdim=128, block=4096),
    "w4096": dict(width=4096, heads=32, layers=4, experts=32, top=4, expert_ff=1536, gla_dim=64, gla_vdim=128, block=4096),
}
DAZILIX_RECURRENT_LAYERS = (2,)


def dazilix_config(s: dict) -> dict:
    att = {"heads": s["heads"], "kv_heads": 8, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "rot": {"base": 1000000.0, "dims": 64},
           "mask": {"size": s["block"]}}
    gla = {"heads": s["heads"], "dim": s["gla_dim"], "vdim": s["gla_vdim"], "tau": 16.0, "decay_rank": 16}
    moe = {"kind": "moe", "router": {"experts": s["experts"], "top": s["top"]}, "expert": {"ff": s["expert_ff"]}}
    return {"architecture": "Dazilix", "vocab": VOCAB, "width": s["width"], "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "layers": [{"type": "gla", "mixer": gla, "mlp": moe} if i in DAZILIX_RECURRENT_LAYERS else {"type": "attention", "mixer": att, "mlp": moe}
                       for i in range(s["layers"])]}


def qwen3_beside_dazilix(s: dict) -> dict:
    inter = int(round(s["top"] * s["expert_ff"] / 64)) * 64  # SwiGLU of the same weight per token as the chosen experts
    return {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": s["layers"], "hidden_size": s["width"],
            "num_attention_heads": s["heads"], "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": inter, "vocab_size": VOCAB,
            "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 8192,
            "hidden_act": "silu", "attention_bias": False, "torch_dtype": "bfloat16"}


# Pekunex at the same widths: a capped attention, the pair side by side (attention with sinks beside a matrix memory whose
# state is [heads, 64, 128 + 1] float32 per request), a state-space layer (inner width twice the model's, state 128) and a
# second capped attention; heads of 128; a dense SwiGLU of the weight per token of Dazilix's chosen experts.
PEKUNEX_SIZES = {
    "w2048": dict(width=2048, heads=16, layers=4, ff=2048, mem_dim=64, mem_vdim=128, ssm_heads=64, ssm_vdim=64, ssm_state=128, ssm_groups=8),
    "w4096": dict(width=4096, heads=32, layers=4, ff=6144, mem_dim=64, mem_vdim=128, ssm_heads=128, ssm_vdim=64, ssm_state=128, ssm_groups=8),
}


def pekunex_config(s: dict) -> dict:
    att = {"heads": s["heads"], "kv_heads": 8, "dim": 128, "vdim": 128, "scale": 1.0, "softcap": 30.0,
           "rot": {"base": 1000000.0, "dims": 64, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    left = {"heads": s["heads"], "kv_heads": 8, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
            "rot": {"base": 1000000.0, "dims": 128, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 4096}}}
    right = {"heads": s["heads"], "dim": s["mem_dim"], "vdim": s["mem_vdim"], "gate_cap": 15.0}
    ssm = {"heads": s["ssm_heads"], "vdim": s["ssm_vdim"], "state": s["ssm_state"], "groups": s["ssm_groups"], "conv": 4, "norm_groups": 8}
    mlp = {"kind": "dense", "ff": s["ff"]}
    return {"architecture": "Pekunex", "vocab": VOCAB, "width": s["width"], "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0}, "logit_scale": 1.0,
            "layers": [{"type": "attention", "mixer": att, "mlp": mlp},
                       {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": 1.0, "right_scale": 1.0}, "mlp": mlp},
                       {"type": "mamba2", "mixer": ssm, "mlp": mlp}, {"type": "attention", "mixer": att, "mlp": mlp}]}


def dazilix_beside_pekunex(s: dict) -> dict:
    d = next(v for k, v in DAZILIX_SIZES.items() if v["width"] == s["width"])
    return dazilix_config(d)


# Vasosun at the same widths: a windowed attention (heads of 128, a window that holds the prompt, so that it does the work
# of Dazilix's attention), a latent attention (512 + 64 cached per token, queries through a latent of three quarters of the
# width), a second one that reads the first one's rows, and a delta layer whose state is [heads, 64, 128] float32 per request
# as Dazilix's recurrent layer's; routed experts of Dazilix's sizes (two more router outputs are identity experts).
VASOSUN_SIZES = {
    "w2048": dict(width=2048, heads=16, layers=4, experts=16, top=2, expert_ff=1024, identity=2, delta_dim=64, delta_vdim=128, window=4096,
                  kv_rank=512, rot_dim=64, q_rank=1536, taps=4),
    "w4096": dict(width=4096, heads=32, layers=4, experts=32, top=4, expert_ff=1536, identity=2, delta_dim=64, delta_vdim=128, window=4096,
                  kv_rank=512, rot_dim=64, q_rank=3072, taps=4),
}


def vasosun_config(s: dict) -> dict:
    att = {"heads": s["heads"], "kv_heads": 8, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "mask": {"size": s["window"]},
           "q_temp": {"coef": 0.5, "every": 1024}}
    lat = {"heads": s["heads"], "dim": 128, "rot_dim": s["rot_dim"], "vdim": 128, "kv_rank": s["kv_rank"], "q_rank": s["q_rank"],
           "scale": 192 ** -0.5, "rot": {"base": 1000000.0, "dims": s["rot_dim"],
                                         "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    delta = {"heads": s["heads"], "kv_heads": s["heads"], "dim": s["delta_dim"], "vdim": s["delta_vdim"], "conv": 4}
    moe = {"kind": "moe", "expert": {"ff": s["expert_ff"]}, "router": {"experts": s["experts"], "identity": s["identity"], "top": s["top"]}}
    return {"architecture": "Vasosun", "vocab": VOCAB, "width": s["width"], "norm": {"eps": 1e-6}, "canon": {"taps": s["taps"]},
            "embedding": {"bigram": {"buckets": 65521, "mul_prev": 1000003, "mul_cur": 31}}, "logit_softcap": 30.0,
            "layers": [{"type": "attention", "mixer": att, "mlp": moe}, {"type": "latent_attention", "mixer": lat, "mlp": moe},
                       {"type": "latent_attention", "mixer": dict(lat, kv_from=1), "mlp": moe}, {"type": "delta", "mixer": delta, "mlp": moe}]}


def dazilix_beside_vasosun(s: dict) -> dict:
    d = next(v for k, v in DAZILIX_SIZES.items() if v["width"] == s["width"])
    return dazilix_config(d)


def _vasosun_rooflines(s: dict, m: dict, peaks: dict) -> dict[str, Any]:
    """Vasosun's recurrence and small kernels against their rooflines, from the per-class timers.  The delta
    rule: a prompt costs 8 float32 operations per state entry and token (decay, two read-outs of the decayed
    state, the update) against the FFMA rate of the SMs at their top clock; a decode step reads and writes every
    request's state once, against the measured copy bandwidth.  The convolutions (two per layer on the normed
    rows, one on q, k, v of the delta layer), the kernels that close a sublayer, and the kernel between the
    attention's projections and attention move their inputs and outputs once, against the same."""
    out: dict[str, Any] = {}
    H, d, e, W, L = s["heads"], s["delta_dim"], s["delta_vdim"], s["width"], s["layers"]
    entries = H * d * e
    ffma_peak = 148 * 128 * 2 * peaks.get("sm_max_mhz", 1965.0) * 1e6
    hbm = peaks["hbm_gbs"] * 1e9
    T = PREFILL_TOKENS
    chans = 2 * H * d + H * e
    small = {
        "causal_conv": 2 * L * W * (2 + 2) + chans * (2 + 4),       # normed rows in and out in bf16, twice a layer; q, k, v in bf16, out float32
        "branch_norm_add": 2 * L * W * 12,                           # the branch (bf16), the stream (float32, read and written), the next input (bf16)
        "qkv_prepare": 2 * (H + 16) * 128 * 2,                       # one attention: q, k, v read and written
        "gla_norm_gate": H * e * (4 + 2 + 2),                        # the read-out float32, gate and result bf16
        "latent_prepare": 2 * (H * 192 * 2 + 576 * 2),               # two latent layers: queries read, rotated parts and the cached row written
    }
    for phase, kernels, tokens in [("prefill", m["prefill_kernels"], T)] + [(f"decode_b{b}", m[f"decode_b{b}_kernels"], b) for b in DECODE_BATCHES]:
        ms = kernels.get("delta_scan", {}).get("ms", 0.0)
        if ms > 0:
            out[f"{phase}_delta_scan_ms"] = round(ms, 4)
            if phase == "prefill":
                out["prefill_delta_scan_of_ffma_peak"] = round(8.0 * T * entries / (ms * 1e-3) / ffma_peak, 3)
            else:
                out[f"{phase}_delta_scan_of_hbm_peak"] = round(tokens * entries * 8 / (ms * 1e-3) / hbm, 3)
        for name, per_token in small.items():
            ms = kernels.get(name, {}).get("ms", 0.0)
            if ms > 0:
                out[f"{phase}_{name}_ms"] = round(ms, 4)
                if phase == "prefill":
                    out[f"prefill_{name}_of_hbm_peak"] = round(tokens * per_token / (ms * 1e-3) / hbm, 3)
    # the latent attention kernel, as Fegetar's is counted: per (query, key, head) 576 + 512 multiply-adds; a decode step reads every cached row once per layer
    ms = m["prefill_kernels"].get("latent_attention_mma", {}).get("ms", 0.0)
    pairs = T * (T + 1) / 2
    if ms > 0:
        out["prefill_latent_attention_ms"] = round(ms, 3)
        out["prefill_latent_attention_of_bf16_peak"] = round(2 * 2 * H * pairs * (576 + 512) / (ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 3)
    for batch in DECODE_BATCHES:
        ms = m[f"decode_b{batch}_kernels"].get("latent_attention_mma", {}).get("ms", 0.0)
        if ms > 0:
            out[f"decode_b{batch}_latent_attention_ms"] = round(ms, 4)
            out[f"decode_b{batch}_latent_attention_of_hbm_peak"] = round(2 * batch * DECODE_CONTEXT * 576 * 2 / (ms * 1e-3) / hbm, 3)
    return out


def _pekunex_rooflines(s: dict, m: dict, peaks: dict) -> dict[str, Any]:
    """Pekunex's recurrences and small kernels against their rooflines, from the per-class timers.  The
    recurrence (both mixers run the same kernel): a prompt costs 6 float32 operations per state entry and
    token against the FFMA rate of the SMs at their top clock; a decode step reads and writes every
    request's states once, against the measured copy bandwidth.  The kernels between the projections
    and attention (biases, rotation, unit norm, store; the gate behind attention) and around the
    recurrences (convolution, gates, norms) move their inputs and outputs once, against the same."""
    out: dict[str, Any] = {}
    H, d, e = s["heads"], s["mem_dim"], s["mem_vdim"] + 1
    Hs, N, es, G = s["ssm_heads"], s["ssm_state"], s["ssm_vdim"], s["ssm_groups"]
    entries = H * d * e + Hs * N * es  # state entries of one request, both recurrent layers
    ffma_peak = 148 * 128 * 2 * peaks.get("sm_max_mhz", 1965.0) * 1e6
    hbm = peaks["hbm_gbs"] * 1e9
    T, W = PREFILL_TOKENS, s["width"]
    inner, chans = Hs * es, Hs * es + 2 * G * N
    # bytes per token of the small kernels (bf16 in and out unless float32 is named)
    small = {
        "qkv_prepare": 3 * 2 * (H + 16) * 128 * 2,                                  # three attentions: q, k, v read and written
        "gate_rows": 2 * 3 * H * 128 * 2,                                              # two gated attentions: heads, gate, result
        "ssm_conv": chans * 2 + chans * 4 + 3 * Hs * 4,                                # inputs bf16, outputs float32, step sizes and decays
        "ssm_gate_norm": inner * (4 + 4 + 2 + 2),                                      # read-out and x float32, z and result bf16
        "mlstm_norm_gate": H * e * 4 + 2 * H * (e - 1) * 2,                            # read-out float32, gate and result bf16
        "weighted_sum": 3 * W * 2,
    }
    for phase, kernels, tokens in [("prefill", m["prefill_kernels"], T)] + [(f"decode_b{b}", m[f"decode_b{b}_kernels"], b) for b in DECODE_BATCHES]:
        ms = kernels.get("linear_scan", {}).get("ms", 0.0)
        if ms > 0:
            out[f"{phase}_linear_scan_ms"] = round(ms, 4)
            if phase == "prefill":
                out["prefill_linear_scan_of_ffma_peak"] = round(6.0 * T * entries / (ms * 1e-3) / ffma_peak, 3)
            else:
                out[f"{phase}_linear_scan_of_hbm_peak"] = round(tokens * entries * 8 / (ms * 1e-3) / hbm, 3)
        for name, per_token in small.items():
            ms = kernels.get(name, {}).get("ms", 0.0)
            if ms > 0:
                out[f"{phase}_{name}_ms"] = round(ms, 4)
                if phase == "prefill":
                    out[f"prefill_{name}_of_hbm_peak"] = round(tokens * per_token / (ms * 1e-3) / hbm, 3)
    return out


def _random_ids(n: int, seed: int) -> list[int]:
    import torch

    return torch.randint(0, VOCAB, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _measure(model, steps: int, warmup: int) -> dict[str, Any]:
    import torch

    from tokensprint_b200 import ops
    from tokensprint_b200.engine.runner import ModelRunner, StepEntry

    out: dict[str, Any] = {}
    pages = max(DECODE_BATCHES) * (-(-(DECODE_CONTEXT + warmup + steps + 8) // PAGE)) + PREFILL_TOKENS // PAGE + 16
    runner = ModelRunner(model, page_size=PAGE, num_pages=pages, num_slots=max(DECODE_BATCHES), max_num_batched_tokens=8192,
                         enforce_eager=False, max_model_len=DECODE_CONTEXT + warmup + steps + 64)
    cm = runner.cache_manager

    def prefill_once(seed: int) -> float:
        rc = cm.admit(("prefill", seed))
        cm.extend(rc, 0, PREFILL_TOKENS)
        entry = StepEntry(rc, _random_ids(PREFILL_TOKENS, seed), 0, [PREFILL_TOKENS - 1])
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        runner.step([entry])
        b.record()
        torch.cuda.synchronize()
        runner.free(rc)
        return a.elapsed_time(b)

    times = sorted(prefill_once(r) for r in range(7))[1:-1]
    out["prefill_ms"] = round(times[len(times) // 2], 3)
    out["prefill_tokens_per_s"] = round(PREFILL_TOKENS / out["prefill_ms"] * 1e3)
    ops.time_kernels(True)
    ops.kernel_times()
    prefill_once(99)
    out["prefill_kernels"] = ops.kernel_times()
    ops.time_kernels(False)

    for batch in DECODE_BATCHES:
        reqs = [cm.admit(("decode", batch, b)) for b in range(batch)]
        for i in range(0, batch, 8):
            entries = []
            for b in range(i, min(batch, i + 8)):
                cm.extend(reqs[b], 0, DECODE_CONTEXT)
                entries.append(StepEntry(reqs[b], _random_ids(DECODE_CONTEXT, 100 + b), 0, []))
            runner.step(entries)
        tokens = [_random_ids(warmup + steps + 1, 500 + b) for b in range(batch)]

        def one(i: int) -> None:
            pos = DECODE_CONTEXT + i
            entries = []
            for b in range(batch):
                cm.extend(reqs[b], pos, pos + 1)
                entries.append(StepEntry(reqs[b], [tokens[b][i]], pos, [0]))
            runner.step(entries)

        for i in range(warmup):
            one(i)
        torch.cuda.synchronize()
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(warmup, warmup + steps):
            one(i)
        b_.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b_) / steps
        out[f"decode_b{batch}_ms"] = round(ms, 4)
        out[f"decode_b{batch}_tokens_per_s"] = round(batch / ms * 1e3)
        # one more step launched kernel by kernel, with a timer around every class
        graphs, runner.use_graphs = runner.use_graphs, False
        ops.time_kernels(True)
        ops.kernel_times()
        one(warmup + steps)
        out[f"decode_b{batch}_kernels"] = ops.kernel_times()
        ops.time_kernels(False)
        runner.use_graphs = graphs
        for rc in reqs:
            runner.free(rc)
    out["graphs"] = bool(runner._graphs)
    return out


def _attention_rooflines(design: str, s: dict, m: dict, peaks: dict) -> dict[str, Any]:
    """Achieved / roofline of the attention kernels from the per-class timers (all layers summed)."""
    L, H, T = s["layers"], s["heads"], PREFILL_TOKENS
    pairs = T * (T + 1) / 2
    if design == "fegetar":
        names = ("latent_attention_mma",)
        flops = L * 2 * H * pairs * (576 + 512)
        row_bytes = 576 * 2
    elif design == "pekunex":
        L = 3  # two capped attentions and the attention of the pair
        names = ("attention_prefill_tcgen05", "attention_paged_mma")
        flops = L * 4 * H * 128 * pairs
        row_bytes = 2 * 8 * 128 * 2
    elif design == "vasosun":
        L = 1  # the windowed attention (the latent layers have a kernel of their own)
        names = ("attention_prefill_tcgen05", "attention_paged_mma", "attention_paged_simple")
        flops = L * 4 * H * 128 * pairs
        row_bytes = 2 * 8 * 128 * 2
    elif design == "dazilix":
        L = s["layers"] - len(DAZILIX_RECURRENT_LAYERS)
        names = ("attention_prefill_tcgen05", "attention_paged_mma")
        flops = L * 4 * H * 128 * pairs
        row_bytes = 2 * 8 * 128 * 2
    else:
        names = ("attention_prefill_tcgen05", "attention_paged_mma", "attention_decode_flat")
        flops = L * 4 * H * 128 * pairs
        row_bytes = 2 * 8 * 128 * 2
    out: dict[str, Any] = {}

    def ms_of(kernels: dict) -> float:
        return sum(v["ms"] for k, v in kernels.items() if k in names)

    ms = ms_of(m["prefill_kernels"])
    if ms > 0:
        out["prefill_attention_ms"] = round(ms, 3)
        out["prefill_attention_of_bf16_peak"] = round(flops / (ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 3)
    for batch in DECODE_BATCHES:
        ms = ms_of(m[f"decode_b{batch}_kernels"])
        if ms > 0:
            out[f"decode_b{batch}_attention_ms"] = round(ms, 4)
            out[f"decode_b{batch}_attention_of_hbm_peak"] = round(L * batch * DECODE_CONTEXT * row_bytes / (ms * 1e-3) / (peaks["hbm_gbs"] * 1e9), 3)
    return out


def _dazilix_rooflines(s: dict, m: dict, peaks: dict) -> dict[str, Any]:
    """The recurrent mixer and the norm kernels of Dazilix against their rooflines, from the per-class
    timers.  The recurrence: a prompt costs 6 float32 operations per state entry and token (decay,
    outer product, read-out) against the FFMA rate of the SMs at their top clock; a decode step reads and
    writes every request's state once, against the measured copy bandwidth.  The norm kernels move
    the branch (bf16), the stream (float32, read and written) and the next sublayer's input (bf16)."""
    out: dict[str, Any] = {}
    L, H, d, e, W = len(DAZILIX_RECURRENT_LAYERS), s["heads"], s["gla_dim"], s["gla_vdim"], s["width"]
    ffma_peak = 148 * 128 * 2 * peaks.get("sm_max_mhz", 1965.0) * 1e6

    def ms_of(kernels: dict, name: str) -> float:
        return kernels.get(name, {}).get("ms", 0.0)

    ms = ms_of(m["prefill_kernels"], "gla_scan")
    if ms > 0:
        out["prefill_gla_scan_ms"] = round(ms, 3)
        out["prefill_gla_scan_of_ffma_peak"] = round(L * 6.0 * PREFILL_TOKENS * H * d * e / (ms * 1e-3) / ffma_peak, 3)
    ms = ms_of(m["prefill_kernels"], "branch_norm_add")
    if ms > 0:
        out["prefill_norms_of_hbm_peak"] = round(2 * s["layers"] * PREFILL_TOKENS * W * 12 / (ms * 1e-3) / (peaks["hbm_gbs"] * 1e9), 3)
    for batch in DECODE_BATCHES:
        ms = ms_of(m[f"decode_b{batch}_kernels"], "gla_scan")
        if ms > 0:
            out[f"decode_b{batch}_gla_scan_ms"] = round(ms, 4)
            out[f"decode_b{batch}_gla_scan_of_hbm_peak"] = round(L * batch * H * d * e * 8 / (ms * 1e-3) / (peaks["hbm_gbs"] * 1e9), 3)
    return out


def _qwen3_norm_roofline(s: dict, m: dict, peaks: dict) -> dict[str, Any]:
    ms = m["prefill_kernels"].get("add_rmsnorm", {}).get("ms", 0.0)
    if ms <= 0:
        return {}
    # per layer two kernels that move the branch (bf16), the stream (float32, read and written) and the normed rows (bf16)
    return {"prefill_norms_of_hbm_peak": round(2 * s["layers"] * PREFILL_TOKENS * s["width"] * 12 / (ms * 1e-3) / (peaks["hbm_gbs"] * 1e9), 3)}


def run(steps: int, warmup: int, peaks: dict, which: str = "fegetar") -> dict[str, Any]:
    import gc

    import torch

    from tokensprint_b200.config.registry import architecture_for
    from tokensprint_b200.models.api import random_model

    result: dict[str, Any] = {"metric": "design_comparison", "dtype": "bf16", "data": "synthetic, random weights",
                              "prefill_tokens": PREFILL_TOKENS, "decode_context": DECODE_CONTEXT, "sizes": {}}
    sizes = {"dazilix": DAZILIX_SIZES, "pekunex": PEKUNEX_SIZES, "vasosun": VASOSUN_SIZES}.get(which, SIZES)
    for name, s in sizes.items():
        row: dict[str, Any] = {"size": s}
        if which == "vasosun":
            pair = (("vasosun", vasosun_config(s)), ("dazilix", dazilix_beside_vasosun(s)))
        elif which == "pekunex":
            pair = (("pekunex", pekunex_config(s)), ("dazilix", dazilix_beside_pekunex(s)))
        elif which == "dazilix":
            pair = (("dazilix", dazilix_config(s)), ("qwen3", qwen3_beside_dazilix(s)))
        else:
            pair = (("fegetar", fegetar_config(s)), ("qwen3", qwen3_config(s)))
        for design, cfg_dict in pair:
            cfg = architecture_for(cfg_dict).config_from_dict(cfg_dict)
            model = random_model(cfg, seed=1, device="cuda", dtype="bfloat16", generate_on_device=True)
            m = _measure(model, steps, warmup)
            m["weight_bytes"] = model.weight_bytes()
            sd = DAZILIX_SIZES[name] if (which in ("pekunex", "vasosun") and design == "dazilix") else s
            m.update(_attention_rooflines(design, sd, m, peaks))
            if which == "vasosun":
                m.update(_vasosun_rooflines(s, m, peaks) if design == "vasosun" else _dazilix_rooflines(sd, m, peaks))
            elif which == "pekunex":
                m.update(_pekunex_rooflines(s, m, peaks) if design == "pekunex" else _dazilix_rooflines(sd, m, peaks))
            elif which == "dazilix":
                m.update(_dazilix_rooflines(s, m, peaks) if design == "dazilix" else _qwen3_norm_roofline(s, m, peaks))
            row[design] = m
            del model
            gc.collect()
            torch.cuda.empty_cache()
        result["sizes"][name] = row
    return result


