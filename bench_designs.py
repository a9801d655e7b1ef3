"""Designs side by side at equal layer sizes: the Kugilix decoder beside the Qwen2 dense decoder, or (``design`` =
"nusudra" / "netinex") the Nusudra or the Netinex decoder beside both, or (``design`` = "sumevik") the Sumevik decoder
beside the Netinex decoder (the closest existing design: attention within chunks, a linear recurrence, experts) and
Qwen2, random weights.

Called by ``bench.py --designs [--design nusudra|netinex|sumevik]``.  For each of a few sizes that resemble a real model's layers it measures, through
the step function, the prefill of one prompt and decode steps at two batch sizes for both designs, and times the
kernels that only the Kugilix design has (decayed linear attention, the windowed attention with slopes, the short
convolution, the norms in groups, the gated norm, the activation) alone, with what they reach of the measured copy
bandwidth or, where they are bound by fp32 arithmetic, of the nominal fp32 rate.
"""

from __future__ import annotations

import math
import statistics

FP32_NOMINAL_TFLOPS = 80.0  # B200, fp32 FMAs outside the tensor cores (nominal; there is no measured figure)

SIZES = {
    # name: width, heads, kv heads, head size, feed-forward, layers of the Kugilix model (a span of four runs twice)
    "1B-like": dict(width=2048, heads=16, kv_heads=4, dim=128, ff=8192, layers=8),
    "3B-like": dict(width=3072, heads=24, kv_heads=8, dim=128, ff=12288, layers=8),
    "small": dict(width=1024, heads=16, kv_heads=8, dim=64, ff=4096, layers=8),
}
WINDOW = 1024
VOCAB = 32000


def kugilix_config(s: dict) -> dict:
    att = {"type": "attention",
           "mixer": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"],
                     "scale": 1.0 / math.sqrt(s["dim"]), "mask": {"size": WINDOW}, "q_temp": {"coef": 0.3, "every": 128}},
           "mlp": {"kind": "dense", "ff": s["ff"]}}
    lin = {"type": "lightning",
           "mixer": {"heads": s["heads"], "dim": s["dim"], "vdim": s["dim"],
                     "decay": [round(1.0 - 2.0 ** (-2 - 6 * h / s["heads"]), 6) for h in range(s["heads"])]},
           "mlp": {"kind": "dense", "ff": s["ff"]}}
    order = [att, lin, lin, att, lin, lin, att, lin]
    layers = [order[i % len(order)] for i in range(s["layers"])]
    return {"architecture": "Kugilix", "vocab": VOCAB, "width": s["width"], "embedding": {"scale": math.sqrt(s["width"])},
            "norm": {"eps": 1e-6, "groups": 4}, "canon": {"taps": 4}, "layers": layers,
            "loop": {"start": 2, "stop": 6, "times": 2}}


def kugilix_runs(s: dict) -> int:
    return s["layers"] + 4


def qwen2_config(s: dict) -> dict:
    """The closest existing design with as many layer runs, the same width and heads, and a gated feed-forward of as
    many weights as the plain one (three matrices of 2/3 the width), every layer over the same window."""
    inter = (2 * s["ff"] // 3 + 127) // 128 * 128
    n = kugilix_runs(s)
    return {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "vocab_size": VOCAB, "hidden_size": s["width"],
            "intermediate_size": inter, "num_hidden_layers": n, "num_attention_heads": s["heads"],
            "num_key_value_heads": s["kv_heads"], "head_dim": s["dim"], "max_position_embeddings": 8192,
            "rms_norm_eps": 1e-6, "rope_theta": 1e6, "hidden_act": "silu", "tie_word_embeddings": False,
            "use_sliding_window": True, "sliding_window": WINDOW, "max_window_layers": 0}


NUSUDRA_ORDER = ("delta", "latent_attention", "parallel")


def nusudra_config(s: dict) -> dict:
    """As many layers as the Kugilix model has layer runs, its three mixers in turn; the same width, heads, head
    size and feed-forward; four residual streams.  The latent row (192 + 64) is the widest the general attention
    kernel takes; the state-space layer has as many heads of the same size, a state of 128 and one group."""
    H, G, d = s["heads"], s["kv_heads"], s["dim"]
    mixers = {
        "delta": {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "conv": 4},
        "latent_attention": {"heads": H, "dim": d, "rot_dim": 64, "vdim": d, "kv_rank": 192,
                             "scale": 1.0 / math.sqrt(d + 64), "rot": {"base": 10000.0, "dims": 64}},
        "parallel": {"left": {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": 1.0 / math.sqrt(d)},
                     "right": {"heads": H, "vdim": d, "state": 128, "groups": 1, "norm_groups": 1, "conv": 4}},
    }
    layers = [{"type": NUSUDRA_ORDER[i % 3], "mixer": mixers[NUSUDRA_ORDER[i % 3]], "mlp": {"kind": "dense", "ff": s["ff"]}}
              for i in range(kugilix_runs(s))]
    return {"architecture": "Nusudra", "vocab": VOCAB, "width": s["width"], "embedding": {"scale": math.sqrt(s["width"])},
            "norm": {"eps": 1e-6}, "streams": 4, "layers": layers}


EXPERTS, TOP = 8, 2


def netinex_expert_ff(s: dict) -> int:
    """An expert's inner size such that the ``TOP`` experts a token uses hold as many weights as the Kugilix model's
    plain feed-forward (two matrices of ff against TOP x three), in multiples of 64."""
    return max(64, (2 * s["ff"]) // (3 * TOP) // 64 * 64)


def netinex_config(s: dict) -> dict:
    """As many layers as the Kugilix model has layer runs, in its order (an attention, two retentions, ...); the same
    width, heads, head size; chunks as long as the other designs' window; ``TOP`` of ``EXPERTS`` gated experts that
    together hold the weights of the plain feed-forward."""
    H, G, d = s["heads"], s["kv_heads"], s["dim"]
    mlp = {"kind": "moe", "expert": {"ff": netinex_expert_ff(s)}, "router": {"experts": EXPERTS, "top": TOP}}
    att = {"type": "attention",
           "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": 1.0 / math.sqrt(d), "mask": {"size": WINDOW},
                     "rot": {"base": 10000.0, "dims": d,
                             "scaling": {"factor": 4.0, "original": 2048, "fast": 32.0, "slow": 1.0}}},
           "mlp": mlp}
    ret = {"type": "retention",
           "mixer": {"heads": H, "dim": d, "vdim": d, "rot": {"base": 1000000.0, "dims": d},
                     "decay": [round(1.0 - 2.0 ** (-2 - 6 * h / H), 6) for h in range(H)]},
           "mlp": mlp}
    order = [att, ret, ret]
    return {"architecture": "Netinex", "vocab": VOCAB, "width": s["width"], "norm": {"eps": 1e-6}, "logit_softcap": 30.0,
            "layers": [order[i % 3] for i in range(kugilix_runs(s))]}


SUMEVIK_IDENTITY = 2  # router outputs beside the EXPERTS experts that stand for "the token's own row"


def sumevik_dense_ff(s: dict) -> int:
    """The inner size of a gated feed-forward of as many weights as the plain one of ``ff`` (three matrices for two)."""
    return (2 * s["ff"] // 3 + 127) // 128 * 128


def sumevik_config(s: dict) -> dict:
    """As many layers as the Kugilix model has layer runs: two recurrent layers, then an attention beside a gated linear
    attention, and so on; the recurrence as wide as the model with as many gate blocks as heads; the same heads and head
    size, chunks as long as the other designs' window, half of every head rotating; the linear attention with as many
    heads, keys of half and values of the full head size; a gated feed-forward in every second layer, ``TOP`` of
    ``EXPERTS`` experts (+ ``SUMEVIK_IDENTITY`` identity experts, two groups of which one stays) in the others."""
    H, G, d, W = s["heads"], s["kv_heads"], s["dim"], s["width"]
    outputs = EXPERTS + SUMEVIK_IDENTITY
    moe = {"kind": "moe", "expert": {"ff": netinex_expert_ff(s), "limit": 7.0},
           "router": {"experts": EXPERTS, "identity": SUMEVIK_IDENTITY, "top": TOP, "groups": {"count": 2, "keep": 1}}}
    assert outputs % 2 == 0
    dense = {"kind": "dense", "ff": sumevik_dense_ff(s)}
    rec = {"type": "rglru", "mixer": {"width": W, "blocks": H, "conv": 4}}
    par = {"type": "parallel",
           "mixer": {"left": {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": 1.0 / math.sqrt(d),
                              "mask": {"size": WINDOW}, "rot": {"base": 500000.0, "dims": d // 2}},
                     "right": {"heads": H, "dim": d // 2, "vdim": d, "tau": 8.0}, "left_scale": 0.9, "right_scale": 1.2}}
    order = [rec, rec, par]
    layers = [dict(order[i % 3], mlp=moe if i % 2 else dense) for i in range(kugilix_runs(s))]
    return {"architecture": "Sumevik", "vocab": VOCAB, "width": W, "norm": {"eps": 1e-6}, "logit_scale": 0.7, "layers": layers}


def _timed(fn, flush, warmup=3, iters=5, reps=1):
    """Seconds per launch: the median of ``iters`` regions of ``reps`` launches back to back, a buffer larger than L2
    written before each region.  ``reps`` > 1 for kernels of a few microseconds, whose single launch would be timed
    together with the host's way to it; their operands are small and lie in L2 inside a step as well."""
    import torch

    for _ in range(warmup):
        fn()
    times = []
    for _ in range(iters):
        flush.add_(1.0)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / reps)
    return statistics.median(times) * 1e-3


def kernel_numbers(s: dict, peaks: dict) -> dict:
    """The Kugilix design's own kernels alone at the layer sizes ``s``: seconds, and the fraction of the roofline each
    is measured against (``hbm``: bytes that must move over the measured copy bandwidth; ``fp32``: FMAs over the
    nominal fp32 rate)."""
    import torch
    from types import SimpleNamespace

    from ferrisinfer_b200.kernels import ops
    from ferrisinfer_b200.parts.position import DistanceSlopes

    dev = torch.device("cuda")
    bf = torch.bfloat16
    flush = torch.zeros(96 << 20, dtype=torch.float32, device=dev)  # 384 MB
    W, H, G, d, ff = s["width"], s["heads"], s["kv_heads"], s["dim"], s["ff"]
    hbm = peaks["hbm_gbs"] * 1e9
    out = {}

    def ctx_of(q_lens, start):
        S = len(q_lens)
        q_start = [0]
        for n in q_lens:
            q_start.append(q_start[-1] + n)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        return SimpleNamespace(num_tokens=q_start[-1], num_seqs=S, max_q_len=max(q_lens), workspace=None,
                               token_seq=i32([i for i in range(S) for _ in range(q_lens[i])]),
                               positions=i32([start + j for i in range(S) for j in range(q_lens[i])]),
                               seq_q_start=i32(q_start), seq_start_pos=i32([start] * S), seq_state_slot=i32(list(range(S))))

    def record(name, seconds, bytes_=None, flops=None):
        e = {"us": round(seconds * 1e6, 1)}
        if bytes_ is not None:
            e["GBps"] = round(bytes_ / seconds / 1e9, 1)
            e["frac_hbm"] = round(bytes_ / seconds / hbm, 3)
        if flops is not None:
            e["TFLOPs_fp32"] = round(flops / seconds / 1e12, 2)
            e["frac_fp32_nominal"] = round(flops / seconds / (FP32_NOMINAL_TFLOPS * 1e12), 3)
        out[name] = e

    # ---- decayed linear attention
    for name, q_lens in (("linear_attention_decode_b64", [1] * 64), ("linear_attention_prefill_2048", [2048])):
        T, S = sum(q_lens), len(q_lens)
        proj = torch.randn(T, 4 * H * d, device=dev).to(bf)
        state = torch.zeros(S + 1, H, d, d, device=dev)
        o = torch.empty(T, H * d, device=dev)
        decay = torch.full((H,), 0.97, device=dev)
        ctx = ctx_of(q_lens, 0)
        t = _timed(lambda: ops.linear_attention(proj, (0, H * d, 2 * H * d), o, state, decay, ctx, H, d, d, silu=True), flush)
        moved = 2 * S * H * d * d * 4 + T * 3 * H * d * 2 + T * H * d * 4
        record(name, t, bytes_=moved, flops=4.0 * T * H * d * d)
    # ---- windowed attention with unit-norm keys and slopes
    slopes = DistanceSlopes(8.0).score_slopes(H, dev)
    for name, batch, q_len, ctx_len in (("window_attention_decode_b64", 64, 1, 2048), ("window_attention_prefill_2048", 1, 2048, 0)):
        T = batch * q_len
        pages_each = (ctx_len + q_len + 15) // 16
        k = torch.randn(batch * pages_each + 1, G, 16, d, device=dev).to(bf)
        v = torch.randn_like(k)
        tables = torch.arange(batch * pages_each, dtype=torch.int32, device=dev).view(batch, pages_each)
        qkv = torch.randn(T, (H + 2 * G) * d, device=dev).to(bf)
        o = torch.empty(T, H * d, dtype=bf, device=dev)
        ctx = ctx_of([q_len] * batch, ctx_len)
        t = _timed(lambda: ops.paged_attention_simt(qkv, o, k, v, tables, ctx.token_seq, ctx.positions, H, G, d, WINDOW,
                                                    1.0 / math.sqrt(d), score_slopes=slopes, v_head_dim=d,
                                                    max_q_len=q_len), flush)
        keys = sum(min(WINDOW, ctx_len + j + 1) for j in range(q_len)) * batch
        if q_len == 1:
            record(name, t, bytes_=batch * G * min(WINDOW, ctx_len + 1) * 2 * d * 2 + T * H * d * 4, flops=4.0 * keys * H * d)
        else:
            record(name, t, flops=4.0 * keys * H * d)
        slots = (tables[ctx.token_seq.long(), (ctx.positions // 16).long()] * 16 + ctx.positions % 16).int()
        t = _timed(lambda: ops.qk_prepare_cache_write(qkv, ctx.positions, slots, k, v, H, G, d, d, 1e-6, (0.3, 128)), flush,
                   reps=10)
        record(name.replace("window_attention", "qk_prepare"), t, bytes_=T * (2 * H * d + 4 * G * d) * 2)
    # ---- row-wise kernels of a long step and of a decode step
    for tag, T in (("2048", 2048), ("b64", 64)):
        h = torch.randn(T, W, device=dev)
        w1, w2 = torch.ones(W, device=dev), torch.ones(W, device=dev)
        a, b = torch.empty(T, W, dtype=bf, device=dev), torch.empty(T, W, dtype=bf, device=dev)
        t = _timed(lambda: ops.grouped_rmsnorm_pair(h, w1, w2, 1e-6, 4, a, b), flush, reps=10 if T <= 64 else 1)
        record(f"norm_pair_{tag}", t, bytes_=T * W * (4 + 2 + 2))
        cw = torch.randn(W, 4, device=dev) * 0.1
        cs = torch.zeros(T + 1, 3, W, device=dev)
        ctx = ctx_of([T], 0) if T > 64 else ctx_of([1] * T, 5)
        t = _timed(lambda: ops.short_conv(a, b, cw, cs, ctx), flush, reps=10 if T <= 64 else 1)
        record(f"short_conv_{tag}", t, bytes_=T * W * 4 + (ctx.num_seqs * 3 * W * 8 if T <= 64 else 0))
        z = torch.randn(T, ff, device=dev).to(bf)
        pq = torch.tensor([0.3, -0.2], device=dev)
        t = _timed(lambda: ops.activation(z, z, "xielu", pq), flush, reps=10 if T <= 64 else 1)
        record(f"xielu_{tag}", t, bytes_=T * ff * 4)
        o = torch.randn(T, H * d, device=dev)
        g = torch.randn(T, H * d, device=dev).to(bf)
        y = torch.empty(T, H * d, dtype=bf, device=dev)
        nw = torch.ones(H * d, device=dev)
        t = _timed(lambda: ops.gated_rmsnorm(o, g, nw, 1e-6, y), flush, reps=10 if T <= 64 else 1)
        record(f"gated_norm_{tag}", t, bytes_=T * H * d * (4 + 2 + 2))
    return out


def nusudra_kernel_numbers(s: dict, peaks: dict) -> dict:
    """The Nusudra design's own kernels alone at the layer sizes ``s``, measured as ``kernel_numbers`` measures."""
    import torch
    from types import SimpleNamespace

    from ferrisinfer_b200.engine.workspace import Workspace
    from ferrisinfer_b200.kernels import ops

    dev = torch.device("cuda")
    bf = torch.bfloat16
    flush = torch.zeros(96 << 20, dtype=torch.float32, device=dev)  # 384 MB
    W, H, G, d = s["width"], s["heads"], s["kv_heads"], s["dim"]
    hbm = peaks["hbm_gbs"] * 1e9
    ws = Workspace(dev)
    out = {}

    def ctx_of(q_lens, start):
        S = len(q_lens)
        q_start = [0]
        for n in q_lens:
            q_start.append(q_start[-1] + n)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        return SimpleNamespace(num_tokens=q_start[-1], num_seqs=S, max_q_len=max(q_lens), workspace=ws,
                               max_kv_len=start + max(q_lens),
                               token_seq=i32([i for i in range(S) for _ in range(q_lens[i])]),
                               positions=i32([start + j for i in range(S) for j in range(q_lens[i])]),
                               seq_q_start=i32(q_start), seq_start_pos=i32([start] * S), seq_state_slot=i32(list(range(S))))

    def record(name, seconds, bytes_=None, flops=None):
        e = {"us": round(seconds * 1e6, 1)}
        if bytes_ is not None:
            e["GBps"] = round(bytes_ / seconds / 1e9, 1)
            e["frac_hbm"] = round(bytes_ / seconds / hbm, 3)
        if flops is not None:
            e["TFLOPs_fp32"] = round(flops / seconds / 1e12, 2)
            e["frac_fp32_nominal"] = round(flops / seconds / (FP32_NOMINAL_TFLOPS * 1e12), 3)
        out[name] = e

    # ---- the recurrences: delta rule (q/k heads shared by heads / G value heads) and the state-space form (state 128)
    for form, qk_heads, n, delta in (("delta_rule", G, d, True), ("state_space", 1, 128, False)):
        for tag, q_lens in (("decode_b64", [1] * 64), ("prefill_2048", [2048])):
            T, S = sum(q_lens), len(q_lens)
            q = (torch.randn(T, qk_heads * n, device=dev) / math.sqrt(n)).to(bf)
            k = (torch.randn(T, qk_heads * n, device=dev) / math.sqrt(n)).to(bf)
            v = torch.randn(T, H * d, device=dev).to(bf)
            decay, beta = torch.full((T, H), 0.97, device=dev), torch.full((T, H), 0.5, device=dev)
            state = torch.zeros(S + 1, H, d, n, device=dev)
            o = torch.empty(T, H * d, device=dev)
            ctx = ctx_of(q_lens, 0)
            t = _timed(lambda: ops.gated_recurrence(q, k, v, decay, beta, o, state, ctx, H, qk_heads, n, d, delta_rule=delta), flush)
            moved = 2 * S * H * n * d * 4 + T * (2 * qk_heads * n + H * d) * 2 + T * H * d * 4
            record(f"{form}_{tag}", t, bytes_=moved, flops=(6.0 if delta else 4.0) * T * H * n * d)
    # ---- attention with a sink and a logarithmic distance penalty (every key is seen), and over the shared latent
    terms = ops.ScoreTerms(log_r1=torch.full((H,), 0.5, device=dev), log_r2=torch.full((H,), 0.3, device=dev),
                           sink=torch.zeros(H, device=dev))
    rank, rot = 192, 64
    for name, batch, q_len, ctx_len in (("decode_b64", 64, 1, 2048), ("prefill_2048", 1, 2048, 0)):
        T = batch * q_len
        pages_each = (ctx_len + q_len + 15) // 16
        tables = torch.arange(batch * pages_each, dtype=torch.int32, device=dev).view(batch, pages_each)
        ctx = ctx_of([q_len] * batch, ctx_len)
        keys = sum(ctx_len + j + 1 for j in range(q_len)) * batch
        k = torch.randn(batch * pages_each + 1, G, 16, d, device=dev).to(bf)
        v = torch.randn_like(k)
        qkv = torch.randn(T, (H + 2 * G) * d, device=dev).to(bf)
        o = torch.empty(T, H * d, dtype=bf, device=dev)
        t = _timed(lambda: ops.paged_attention_simt(qkv, o, k, v, tables, ctx.token_seq, ctx.positions, H, G, d, 0,
                                                    1.0 / math.sqrt(d), score_slopes=terms, v_head_dim=d, max_q_len=q_len,
                                                    max_kv_len=ctx_len + q_len, workspace=ws), flush)
        record(f"sink_attention_{name}", t, flops=4.0 * keys * H * d,
               bytes_=batch * G * (ctx_len + 1) * 2 * d * 2 + T * H * d * 4 if q_len == 1 else None)
        kl = torch.randn(batch * pages_each + 1, 1, 16, rank + rot, device=dev).to(bf)
        ql = torch.randn(T, H * (rank + rot), device=dev).to(bf)
        ol = torch.empty(T, H * rank, dtype=bf, device=dev)
        t = _timed(lambda: ops.paged_attention_simt(ql, ol, kl, None, tables, ctx.token_seq, ctx.positions, H, 1, rank + rot, 0,
                                                    0.07, v_head_dim=rank, max_q_len=q_len, max_kv_len=ctx_len + q_len,
                                                    workspace=ws, values_in_keys=True), flush)
        record(f"latent_attention_{name}", t, flops=2.0 * keys * H * (2 * rank + rot),
               bytes_=batch * (ctx_len + 1) * (rank + rot) * 2 + T * H * (2 * rank + rot) * 2 if q_len == 1 else None)
        # the per-head products around it: plain queries through the key up-projection, latents through the value one
        x = torch.randn(T, H * (d + rot), device=dev).to(bf)
        uk = (torch.randn(H, d, rank, device=dev) / math.sqrt(d)).to(bf)
        t = _timed(lambda: ops.head_gemm(x, d + rot, uk, ql, rank + rot), flush, reps=10 if T <= 64 else 1)
        record(f"head_product_{name}", t, flops=2.0 * T * H * d * rank, bytes_=H * d * rank * 2 + T * H * (d + rank) * 2)
        proj = torch.randn(T, H * (d + rot) + rank + rot, device=dev).to(bf)
        slots = (tables[ctx.token_seq.long(), (ctx.positions // 16).long()] * 16 + ctx.positions % 16).int()
        freq = torch.full((rot // 2,), 0.01, device=dev)
        nw = torch.ones(rank, device=dev)
        t = _timed(lambda: ops.latent_prepare(proj, 0, H * (d + rot), nw, 1e-6, ctx.positions, freq, rot, slots, kl, ql, H, d, rot,
                                              rank), flush, reps=10 if T <= 64 else 1)
        record(f"latent_prepare_{name}", t, bytes_=T * (2 * H * rot + 2 * (rank + rot)) * 2)
    # ---- row-wise kernels of a long step and of a decode step
    S4 = 4
    for tag, T in (("2048", 2048), ("b64", 64)):
        xs = torch.randn(T, S4 * W, device=dev)
        y = torch.randn(T, W, device=dev)
        mix, ow, iw, nw = torch.eye(S4, device=dev), torch.ones(S4, device=dev), torch.full((S4,), 0.25, device=dev), torch.ones(W, device=dev)
        a, b = torch.empty(T, W, dtype=bf, device=dev), torch.empty(T, W, dtype=bf, device=dev)
        reps = 10 if T <= 64 else 1
        t = _timed(lambda: ops.streams_step(xs, S4, write=(y, mix, ow), read=(iw, nw, 1e-6, a)), flush, reps=reps)
        record(f"streams_write_read_{tag}", t, bytes_=T * W * (2 * S4 * 4 + 4 + 2))
        ctx = ctx_of([T], 0) if T > 64 else ctx_of([1] * T, 5)
        st = torch.zeros(T + 1, W, device=dev)
        sh = torch.full((W,), 0.3, device=dev)
        t = _timed(lambda: ops.token_shift(a, b, sh, st, ctx), flush, reps=reps)
        record(f"token_shift_{tag}", t, bytes_=T * W * 4 + (T * W * 8 if T <= 64 else 0))
        C = (2 * G + H) * d
        wide = torch.randn(T, C + 64, device=dev).to(bf)
        conv = torch.empty(T, C, dtype=bf, device=dev)
        cw = torch.randn(C, 4, device=dev) * 0.1
        cs = torch.zeros(T + 1, 3, C, device=dev)
        t = _timed(lambda: ops.short_conv(wide[:, :C], conv, cw, cs, ctx, residual=False, silu=True), flush, reps=reps)
        record(f"conv_silu_{tag}", t, bytes_=T * C * 4 + (ctx.num_seqs * 3 * C * 8 if T <= 64 else 0))
        o = torch.randn(T, H * d, device=dev)
        g = torch.randn(T, H * d, device=dev).to(bf)
        yy = torch.empty(T, H * d, dtype=bf, device=dev)
        t = _timed(lambda: ops.gated_group_norm(o, g, torch.ones(d, device=dev), 1e-6, yy, group=d, gate_kind="silu"), flush, reps=reps)
        record(f"gated_head_norm_{tag}", t, bytes_=T * H * d * (4 + 2 + 2))
        ya, yb = torch.randn(T, W, device=dev), torch.randn(T, W, device=dev)
        t = _timed(lambda: ops.branch_norm_sum(y, [(ya, nw), (yb, nw)], 0.5, 1e-6), flush, reps=reps)
        record(f"branch_norm_sum_{tag}", t, bytes_=T * W * 4 * 4)
    return out


def netinex_kernel_numbers(s: dict, peaks: dict) -> dict:
    """The Netinex design's own kernels alone at the layer sizes ``s``, measured as ``kernel_numbers`` measures; the
    experts beside the plain feed-forward of as many weights per token (``bf16``: FLOPs over the measured cuBLAS rate)."""
    import torch
    from types import SimpleNamespace

    from ferrisinfer_b200.engine.workspace import Workspace
    from ferrisinfer_b200.kernels import ops

    dev = torch.device("cuda")
    bf = torch.bfloat16
    flush = torch.zeros(96 << 20, dtype=torch.float32, device=dev)  # 384 MB
    W, H, G, d, ff = s["width"], s["heads"], s["kv_heads"], s["dim"], s["ff"]
    hbm = peaks["hbm_gbs"] * 1e9
    tensor = peaks["bf16_tflops"] * 1e12
    ws = Workspace(dev)
    out = {}

    def ctx_of(q_lens, start):
        S = len(q_lens)
        q_start = [0]
        for n in q_lens:
            q_start.append(q_start[-1] + n)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        return SimpleNamespace(num_tokens=q_start[-1], num_seqs=S, max_q_len=max(q_lens), workspace=ws,
                               max_kv_len=start + max(q_lens),
                               token_seq=i32([i for i in range(S) for _ in range(q_lens[i])]),
                               positions=i32([start + j for i in range(S) for j in range(q_lens[i])]),
                               seq_q_start=i32(q_start), seq_start_pos=i32([start] * S), seq_state_slot=i32(list(range(S))))

    def record(name, seconds, bytes_=None, flops=None, tensor_flops=None):
        e = {"us": round(seconds * 1e6, 1)}
        if bytes_ is not None:
            e["GBps"] = round(bytes_ / seconds / 1e9, 1)
            e["frac_hbm"] = round(bytes_ / seconds / hbm, 3)
        if flops is not None:
            e["TFLOPs_fp32"] = round(flops / seconds / 1e12, 2)
            e["frac_fp32_nominal"] = round(flops / seconds / (FP32_NOMINAL_TFLOPS * 1e12), 3)
        if tensor_flops is not None:
            e["TFLOPs_bf16"] = round(tensor_flops / seconds / 1e12, 1)
            e["frac_bf16_measured"] = round(tensor_flops / seconds / tensor, 3)
        out[name] = e

    # ---- retention: the decayed linear attention with q and k rotated and k scaled on the way in
    freq = torch.exp(-math.log(1e6) * torch.arange(d // 2, device=dev, dtype=torch.float32) * 2 / d)
    table = ops.RotaryTable(freq, d, interleaved=False)
    for name, q_lens in (("retention_decode_b64", [1] * 64), ("retention_prefill_2048", [2048])):
        T, S = sum(q_lens), len(q_lens)
        proj = torch.randn(T, 4 * H * d, device=dev).to(bf)
        state = torch.zeros(S + 1, H, d, d, device=dev)
        o = torch.empty(T, H * d, device=dev)
        decay = torch.full((H,), 0.97, device=dev)
        ctx = ctx_of(q_lens, 7)
        t = _timed(lambda: ops.linear_attention(proj, (0, H * d, 2 * H * d), o, state, decay, ctx, H, d, d, silu=False,
                                                rotary=table, k_scale=d ** -0.5), flush)
        moved = 2 * S * H * d * d * 4 + T * 3 * H * d * 2 + T * H * d * 4
        record(name, t, bytes_=moved, flops=4.0 * T * H * d * d)
    # ---- attention within chunks, the values read from the raw keys' rows; and the kernel ahead of it
    itab = ops.RotaryTable(freq, d, interleaved=True, magnitude=1.1)
    for name, batch, q_len, ctx_len in (("decode_b64", 64, 1, 2047), ("prefill_2048", 1, 2048, 0)):
        T = batch * q_len
        pages_each = (ctx_len + q_len + 15) // 16
        k = torch.randn(batch * pages_each + 1, G, 16, d, device=dev).to(bf)
        v = torch.randn_like(k)
        tables = torch.arange(batch * pages_each, dtype=torch.int32, device=dev).view(batch, pages_each)
        qk = torch.randn(T, (H + G) * d, device=dev).to(bf)
        o = torch.empty(T, H * d, dtype=bf, device=dev)
        ctx = ctx_of([q_len] * batch, ctx_len)
        t = _timed(lambda: ops.paged_attention_simt(qk, o, k, v, tables, ctx.token_seq, ctx.positions, H, G, d, 0,
                                                    1.0 / math.sqrt(d), v_head_dim=d, max_q_len=q_len,
                                                    max_kv_len=ctx_len + q_len, workspace=ws, chunk=WINDOW), flush)
        keys = sum((ctx_len + j) % WINDOW + 1 for j in range(q_len)) * batch
        record(f"chunk_attention_{name}", t, flops=4.0 * keys * H * d,
               bytes_=batch * G * (ctx_len % WINDOW + 1) * 2 * d * 2 + T * H * d * 4 if q_len == 1 else None)
        slots = (tables[ctx.token_seq.long(), (ctx.positions // 16).long()] * 16 + ctx.positions % 16).int()
        qn, kn = torch.ones(H * d, device=dev), torch.ones(G * d, device=dev)
        t = _timed(lambda: ops.qk_norm_rotary_cache_write(qk, ctx, slots, k, v, H, G, d, d, qn, kn, 1e-6, itab,
                                                          values_from_keys=True), flush, reps=10)
        record(f"qk_norm_rotary_{name}", t, bytes_=T * (2 * H * d + 3 * G * d) * 2)
    # ---- row-wise kernels of a long step and of a decode step
    for tag, T in (("2048", 2048), ("b64", 64)):
        reps = 10 if T <= 64 else 1
        h = torch.randn(T, W, device=dev)
        w1, b1, alpha = torch.ones(W, device=dev), torch.zeros(W, device=dev), torch.full((1,), 0.7, device=dev)
        a = torch.empty(T, W, dtype=bf, device=dev)
        t = _timed(lambda: ops.dynamic_tanh(h, w1, b1, alpha, a), flush, reps=reps)
        record(f"dynamic_tanh_{tag}", t, bytes_=T * W * (4 + 2))
        o = torch.randn(T, H * d, device=dev)
        g = torch.randn(T, H * d, device=dev).to(bf)
        y = torch.empty(T, H * d, dtype=bf, device=dev)
        one = torch.ones(1, device=dev)
        t = _timed(lambda: ops.gated_group_norm(o, g, one, 1e-6, y, group=d, gate_kind="silu"), flush, reps=reps)
        record(f"head_norm_silu_gate_{tag}", t, bytes_=T * H * d * (4 + 2 + 2))
        logits = torch.randn(T, VOCAB, device=dev)
        t = _timed(lambda: ops.softcap_(logits, 30.0), flush, reps=reps)
        record(f"softcap_{tag}", t, bytes_=T * VOCAB * 8)
    # ---- the experts beside the plain feed-forward of as many weights per token
    eff = netinex_expert_ff(s)
    gate_up = (torch.randn(EXPERTS, 2 * eff, W, device=dev) / math.sqrt(W)).to(bf)
    down = (torch.randn(EXPERTS, W, eff, device=dev) / math.sqrt(eff)).to(bf)
    router = torch.randn(EXPERTS, W, device=dev).to(bf)
    rb = torch.zeros(EXPERTS, device=dev)
    w_up = (torch.randn(ff, W, device=dev) / math.sqrt(W)).to(bf)
    w_down = (torch.randn(W, ff, device=dev) / math.sqrt(ff)).to(bf)
    for tag, T in (("b8", 8), ("b64", 64), ("2048", 2048)):
        x = torch.randn(T, W, device=dev).to(bf)
        hrow = torch.zeros(T, W, device=dev)
        ids = torch.empty(T, TOP, dtype=torch.int32, device=dev)
        wts = torch.empty(T, TOP, device=dev)
        t = _timed(lambda: ops.moe_router(x, router, rb, ids, wts, TOP), flush, reps=10)
        record(f"router_{tag}", t, bytes_=T * W * 2 + EXPERTS * W * 2)
        distinct = int(torch.unique(ids).numel())
        t = _timed(lambda: ops.moe_experts(x, gate_up, down, ids, wts, hrow, ws, accumulate=True), flush)
        record(f"experts_{tag}", t, bytes_=distinct * 3 * W * eff * 2 + T * W * (2 + 8),
               tensor_flops=2.0 * T * TOP * 3 * W * eff)
        out[f"experts_{tag}"]["distinct_experts"] = distinct
        act = torch.empty(T, ff, dtype=bf, device=dev)

        def dense():
            ops.gemm_activation(x, w_up, act, "silu")
            ops.gemm(act, w_down, None, hrow, accumulate=True)

        t = _timed(dense, flush)
        record(f"dense_feed_forward_{tag}", t, bytes_=2 * W * ff * 2 + T * W * (2 + 8), tensor_flops=2.0 * T * 2 * W * ff)
    return out


def sumevik_kernel_numbers(s: dict, peaks: dict) -> dict:
    """The Sumevik design's own kernels alone at the layer sizes ``s``, measured as ``kernel_numbers`` measures; its gated
    products beside the SiLU-gated ones, its router and experts beside the Netinex design's."""
    import torch
    from types import SimpleNamespace

    from ferrisinfer_b200.engine.workspace import Workspace
    from ferrisinfer_b200.kernels import ops

    dev = torch.device("cuda")
    bf = torch.bfloat16
    flush = torch.zeros(96 << 20, dtype=torch.float32, device=dev)  # 384 MB
    W, H, G, d, ff = s["width"], s["heads"], s["kv_heads"], s["dim"], s["ff"]
    hbm = peaks["hbm_gbs"] * 1e9
    tensor = peaks["bf16_tflops"] * 1e12
    ws = Workspace(dev)
    out = {}

    def ctx_of(q_lens, start):
        S = len(q_lens)
        q_start = [0]
        for n in q_lens:
            q_start.append(q_start[-1] + n)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        return SimpleNamespace(num_tokens=q_start[-1], num_seqs=S, max_q_len=max(q_lens), workspace=ws,
                               max_kv_len=start + max(q_lens),
                               token_seq=i32([i for i in range(S) for _ in range(q_lens[i])]),
                               positions=i32([start + j for i in range(S) for j in range(q_lens[i])]),
                               seq_q_start=i32(q_start), seq_start_pos=i32([start] * S), seq_state_slot=i32(list(range(S))))

    def record(name, seconds, bytes_=None, flops=None, tensor_flops=None):
        e = {"us": round(seconds * 1e6, 1)}
        if bytes_ is not None:
            e["GBps"] = round(bytes_ / seconds / 1e9, 1)
            e["frac_hbm"] = round(bytes_ / seconds / hbm, 3)
        if flops is not None:
            e["TFLOPs_fp32"] = round(flops / seconds / 1e12, 2)
            e["frac_fp32_nominal"] = round(flops / seconds / (FP32_NOMINAL_TFLOPS * 1e12), 3)
        if tensor_flops is not None:
            e["TFLOPs_bf16"] = round(tensor_flops / seconds / 1e12, 1)
            e["frac_bf16_measured"] = round(tensor_flops / seconds / tensor, 3)
        out[name] = e

    # ---- the recurrent unit: gates (block-diagonal products, sigmoids, decay) and the scan over channels
    C, blocks = W, H
    bs = C // blocks
    wa = (torch.randn(blocks, bs, bs, device=dev) / math.sqrt(bs)).to(bf)
    wi = (torch.randn(blocks, bs, bs, device=dev) / math.sqrt(bs)).to(bf)
    ba, bi, rate = torch.zeros(C, device=dev), torch.zeros(C, device=dev), torch.full((C,), 0.05, device=dev)
    for tag, q_lens in (("decode_b64", [1] * 64), ("prefill_2048", [2048])):
        T, S = sum(q_lens), len(q_lens)
        reps = 10 if T <= 64 else 1
        u = torch.randn(T, C, device=dev).to(bf)
        ybranch = torch.randn(T, C, device=dev).to(bf)
        a, b = torch.empty(T, C, device=dev), torch.empty(T, C, device=dev)
        y = torch.empty(T, C, dtype=bf, device=dev)
        state = torch.zeros(S + 1, C, device=dev)
        ctx = ctx_of(q_lens, 5)
        t = _timed(lambda: ops.rglru_gates(u, wa, wi, ba, bi, rate, a, b, 8.0), flush, reps=reps)
        record(f"recurrent_gates_{tag}", t, bytes_=2 * C * bs * 2 + T * C * (2 + 8), flops=2.0 * T * 2 * C * bs)
        if T >= ops.RGLRU_TENSOR_CORE_MIN_TOKENS:  # the form a long bf16 step takes: the products on the tensor cores
            stored = (wa.transpose(1, 2).contiguous(), wi.transpose(1, 2).contiguous())
            t = _timed(lambda: ops.rglru_gates(u, wa, wi, ba, bi, rate, a, b, 8.0, stored=stored), flush, reps=reps)
            record(f"recurrent_gates_tensor_cores_{tag}", t, bytes_=2 * C * bs * 2 + T * C * (2 + 8),
                   tensor_flops=2.0 * T * 2 * C * bs)
        a.uniform_(-0.5, 0.0)  # (in case the gates left something else: the scan takes logarithms of decays)
        t = _timed(lambda: ops.rglru_scan(a, b, ybranch, y, state, ctx), flush, reps=reps)
        record(f"recurrent_scan_{tag}", t, bytes_=T * C * (8 + 2 + 2) + 2 * S * C * 4)
        cw = torch.randn(C, 4, device=dev) * 0.1
        cb = torch.zeros(C, device=dev)
        hist = torch.zeros(S + 1, 3, C, device=dev)
        wide = torch.randn(T, 2 * C, device=dev).to(bf)
        t = _timed(lambda: ops.short_conv(wide[:, C:], u, cw, hist, ctx, bias=cb, residual=False), flush, reps=reps)
        record(f"recurrent_conv_{tag}", t, bytes_=T * C * 4 + (S * 3 * C * 8 if T <= 64 else 0))
    # ---- the gated linear attention: the recurrence with a decay per key channel, and the norm per head with its gate
    dk = d // 2
    for tag, q_lens in (("decode_b64", [1] * 64), ("prefill_2048", [2048])):
        T, S = sum(q_lens), len(q_lens)
        proj = (torch.randn(T, 2 * H * dk + 2 * H * d, device=dev) / 4.0).to(bf)
        z = 3.0 + torch.randn(T, H * dk, device=dev)
        state = torch.zeros(S + 1, H, d, dk, device=dev)
        o = torch.empty(T, H * d, device=dev)
        ctx = ctx_of(q_lens, 0)
        t = _timed(lambda: ops.row_decay_recurrence(proj[:, :H * dk], proj[:, H * dk:2 * H * dk], proj[:, 2 * H * dk:2 * H * dk + H * d],
                                                    z, 1.0 / 8.0, o, state, ctx, H, dk, d, q_scale=dk ** -0.5), flush)
        moved = 2 * S * H * dk * d * 4 + T * (2 * H * dk + H * d) * 2 + T * H * dk * 4 + T * H * d * 4
        record(f"linear_attention_row_decay_{tag}", t, bytes_=moved, flops=4.0 * T * H * dk * d)
    # ---- the attention's own kernels: norm per head + rotation + cache write, the chunked attention with value heads of
    # their own, the gate on its output
    freq = torch.exp(-math.log(1e6) * torch.arange(d // 4, device=dev, dtype=torch.float32) * 4 / d)
    itab = ops.RotaryTable(freq, d // 2, interleaved=True, freq_lo=torch.zeros_like(freq))
    for name, batch, q_len, ctx_len in (("decode_b64", 64, 1, 2047), ("prefill_2048", 1, 2048, 0)):
        T = batch * q_len
        reps = 10 if T <= 64 else 1
        pages_each = (ctx_len + q_len + 15) // 16
        k = torch.randn(batch * pages_each + 1, G, 16, d, device=dev).to(bf)
        v = torch.randn_like(k)
        tables = torch.arange(batch * pages_each, dtype=torch.int32, device=dev).view(batch, pages_each)
        rows = torch.randn(T, (H + 2 * G) * d + H * d, device=dev).to(bf)  # q, k, v and the gate's columns
        qkv, gate = rows[:, :(H + 2 * G) * d], rows[:, (H + 2 * G) * d:]
        o = torch.empty(T, H * d, dtype=bf, device=dev)
        ctx = ctx_of([q_len] * batch, ctx_len)
        slots = (tables[ctx.token_seq.long(), (ctx.positions // 16).long()] * 16 + ctx.positions % 16).int()
        qn, kn = torch.ones(d, device=dev), torch.ones(d, device=dev)
        t = _timed(lambda: ops.qk_norm_rotary_cache_write(qkv, ctx, slots, k, v, H, G, d, d, qn, kn, 1e-6, itab, per_head=True),
                   flush, reps=10)
        record(f"head_norm_rotary_{name}", t, bytes_=T * (2 * H * d + 4 * G * d) * 2)
        t = _timed(lambda: ops.paged_attention_simt(qkv, o, k, v, tables, ctx.token_seq, ctx.positions, H, G, d, 0,
                                                    1.0 / math.sqrt(d), v_head_dim=d, max_q_len=q_len,
                                                    max_kv_len=ctx_len + q_len, workspace=ws, chunk=WINDOW), flush)
        keys = sum((ctx_len + j) % WINDOW + 1 for j in range(q_len)) * batch
        record(f"chunk_attention_{name}", t, flops=4.0 * keys * H * d,
               bytes_=batch * G * (ctx_len % WINDOW + 1) * 2 * d * 2 + T * H * d * 4 if q_len == 1 else None)
        t = _timed(lambda: ops.gate_mul(o, gate, o, "sigmoid", 0.9), flush, reps=reps)
        record(f"output_gate_{name}", t, bytes_=T * H * d * 6)
        og = torch.randn(T, H * d, device=dev)
        yy = torch.empty(T, H * d, dtype=bf, device=dev)
        t = _timed(lambda: ops.gated_group_norm(og, gate, torch.ones(d, device=dev), 1e-6, yy, group=d, gate_kind="silu"), flush, reps=reps)
        record(f"head_norm_silu_gate_{name}", t, bytes_=T * H * d * (4 + 2 + 2))
    # ---- the gated feed-forward: the tanh GELU in the products' epilogues beside the SiLU of the other designs
    inter = sumevik_dense_ff(s)
    gate_up_w = (torch.randn(2 * inter, W, device=dev) / math.sqrt(W)).to(bf)
    for tag, T in (("b8", 8), ("b64", 64), ("2048", 2048)):
        x = torch.randn(T, W, device=dev).to(bf)
        act = torch.empty(T, inter, dtype=bf, device=dev)
        for kind in ("gelu_tanh", "silu"):
            t = _timed(lambda: ops.gemm_gated(x, gate_up_w, act, kind, 0.0, ws), flush)
            record(f"gated_product_{kind}_{tag}", t, bytes_=2 * inter * W * 2 + T * (W + inter) * 2,
                   tensor_flops=2.0 * T * 2 * inter * W)
    # ---- the scored router and the experts with a clamped gate and identity experts
    eff = netinex_expert_ff(s)
    outputs = EXPERTS + SUMEVIK_IDENTITY
    gate_up = (torch.randn(EXPERTS, 2 * eff, W, device=dev) / math.sqrt(W)).to(bf)
    down = (torch.randn(EXPERTS, W, eff, device=dev) / math.sqrt(eff)).to(bf)
    router = torch.randn(outputs, W, device=dev).to(bf)
    corr = torch.zeros(outputs, device=dev)
    for tag, T in (("b8", 8), ("b64", 64), ("2048", 2048)):
        x = torch.randn(T, W, device=dev).to(bf)
        hrow = torch.zeros(T, W, device=dev)
        ids = torch.empty(T, TOP, dtype=torch.int32, device=dev)
        wts = torch.empty(T, TOP, device=dev)
        idw = torch.empty(T, device=dev)
        scored = {"correction": corr, "groups": 2, "keep": 1, "with_weights": EXPERTS, "identity_w": idw}
        t = _timed(lambda: ops.moe_router(x, router, None, ids, wts, TOP, scored=scored), flush, reps=10)
        record(f"scored_router_{tag}", t, bytes_=T * W * 2 + outputs * W * 2)
        chosen = torch.unique(ids)
        distinct = int((chosen < EXPERTS).sum())
        pairs = int((ids < EXPERTS).sum())
        t = _timed(lambda: ops.moe_experts(x, gate_up, down, ids, wts, hrow, ws, accumulate=True, activation="clamped_swish",
                                           limit=7.0, identity_w=idw), flush)
        record(f"experts_clamped_{tag}", t, bytes_=distinct * 3 * W * eff * 2 + T * W * (2 + 8),
               tensor_flops=2.0 * pairs * 3 * W * eff)
        out[f"experts_clamped_{tag}"]["distinct_experts"] = distinct
        out[f"experts_clamped_{tag}"]["pairs_with_weights"] = pairs
    return out


def run(build_engine, time_decode, time_prefill, peaks, steps=32, warmup=4, sizes=("small", "1B-like"), context=2048,
        prompt=2048, batches=(8, 64), kernels_at="1B-like", design="kugilix") -> dict:
    """``build_engine(cfg, batch, context, extra_tokens)``, ``time_decode`` and ``time_prefill`` are bench.py's.
    ``design`` "kugilix": that design beside Qwen2; "nusudra" or "netinex": that design beside both; "sumevik": that
    design beside Netinex and Qwen2."""
    import torch

    result = {"context": context, "prompt_tokens": prompt, "window": WINDOW, "sizes": {}}
    for name in sizes:
        s = SIZES[name]
        entry = {"layer_sizes": s, "layer_runs": kugilix_runs(s)}
        designs = (("kugilix", kugilix_config(s)), ("qwen2", qwen2_config(s)))
        if design == "nusudra":
            designs = (("nusudra", nusudra_config(s)),) + designs
        if design == "netinex":
            designs = (("netinex", netinex_config(s)),) + designs
        if design == "sumevik":
            designs = (("sumevik", sumevik_config(s)), ("netinex", netinex_config(s)), ("qwen2", qwen2_config(s)))
        for design_name, cfg in designs:
            numbers = {}
            engine = build_engine(cfg, 1, context, extra_tokens=prompt)
            ms = time_prefill(engine, prompt)
            numbers["prefill_tok_s"] = round(prompt / ms * 1e3, 1)
            numbers["prefill_ms"] = round(ms, 3)
            del engine
            torch.cuda.empty_cache()
            for b in batches:
                engine = build_engine(cfg, b, context)
                times, launches = time_decode(engine, b, context, steps, warmup, regions=3)
                ms = statistics.median(times)
                numbers[f"decode_b{b}_tok_s"] = round(b / ms * 1e3, 1)
                numbers[f"decode_b{b}_ms"] = round(ms, 4)
                numbers[f"decode_b{b}_launches_per_step"] = launches // steps
                del engine
                torch.cuda.empty_cache()
            entry[design_name] = numbers
        result["sizes"][name] = entry
    if kernels_at and design == "sumevik":
        result["kernels_sumevik"] = {"at": kernels_at, "expert_ff": netinex_expert_ff(SIZES[kernels_at]), "experts": EXPERTS,
                                     "identity": SUMEVIK_IDENTITY, "top": TOP,
                                     **sumevik_kernel_numbers(SIZES[kernels_at], peaks)}
        result["kernels_netinex"] = {"at": kernels_at, "expert_ff": netinex_expert_ff(SIZES[kernels_at]),
                                     "experts": EXPERTS, "top": TOP, **netinex_kernel_numbers(SIZES[kernels_at], peaks)}
    elif kernels_at:
        result["kernels"] = {"at": kernels_at, **kernel_numbers(SIZES[kernels_at], peaks)}
        if design == "nusudra":
            result["kernels_nusudra"] = {"at": kernels_at, **nusudra_kernel_numbers(SIZES[kernels_at], peaks)}
        if design == "netinex":
            result["kernels_netinex"] = {"at": kernels_at, "expert_ff": netinex_expert_ff(SIZES[kernels_at]),
                                         "experts": EXPERTS, "top": TOP,
                                         **netinex_kernel_numbers(SIZES[kernels_at], peaks)}
    return result
