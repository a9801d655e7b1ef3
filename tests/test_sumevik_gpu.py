"""The Sumevik decoder on the GPU against the plain implementation (``plain_sumevik``, float64): each kernel of its
mechanisms alone, then whole models of several small configurations driven through the step function the ways a
server drives it (whole prompts, token by token, portions down to two tokens, mixed batches over pages and state
slots that come back), and greedy generation through the engine."""

import functools
import json
import math
import os
import random

import pytest
import torch

import helpers
import plain_sumevik as plain
import sumevik_cases as cases
from test_netinex_gpu import fake_ctx, paged, tol_of

pytestmark = pytest.mark.gpu
F32, F64, BF16 = torch.float32, torch.float64, torch.bfloat16
DTYPES = {"float32": F32, "bfloat16": BF16}


def _ops():
    from ferrisinfer_b200.kernels import ops
    return ops


def make_runner(cfg, weights, dtype, device, num_pages=24, max_requests=4, graphs=True, page_size=16):
    from ferrisinfer_b200.config import resolve_config
    from ferrisinfer_b200.engine.runner import ModelRunner
    from ferrisinfer_b200.parts import build_model
    from ferrisinfer_b200.weights.loader import bind_tensors

    arch, c = resolve_config(cases.folder_config(cfg))
    model = build_model(arch.plan(c))
    bind_tensors(model, weights, DTYPES[dtype], device)
    return ModelRunner(model, DTYPES[dtype], device, page_size=page_size, num_pages=num_pages, max_requests=max_requests,
                       cuda_graphs=graphs)


@functools.lru_cache(maxsize=None)
def weights_of(case: str):
    return cases.make_weights(cases.CASES[case], seed=sum(map(ord, case)))


@functools.lru_cache(maxsize=None)
def wanted(case: str, n: int, seed: int):
    """(ids, float64 logits of every position) of a random sequence without a close call of any router."""
    return cases.safe_sequence(cases.CASES[case], weights_of(case), n, seed)


def check_rows(got: dict, want: dict, dtype: str, what: str):
    """``want``: request -> float64 logits of every position.  In bfloat16 a few positions amplify rounding several
    times over the typical error: at most one position in fifty may exceed the tolerance, none four times it."""
    worst, where, over, count = 0.0, None, 0, 0
    tol = cases.TOLERANCE[dtype]
    for rid, rows_want in want.items():
        n = rows_want.shape[0]
        rows = torch.stack([got[(rid, p)] for p in range(n)])
        assert torch.isfinite(rows).all(), f"{what}: request {rid} has logits that are not finite"
        err = cases.row_errors(rows, rows_want)
        over, count = over + int((err > tol).sum()), count + n
        if float(err.max()) > worst:
            worst, where = float(err.max()), (rid, int(err.argmax()))
    if dtype == "float32":
        assert worst <= tol, f"{what} ({dtype}): error {worst:.3g} at {where}"
    else:
        assert worst <= 4 * tol and over <= max(1, count // 50), \
            f"{what} ({dtype}): error {worst:.3g} at {where}, {over} of {count} positions over {tol}"


def rounded(w: dict) -> dict:
    """Weights as a folder stores them (bfloat16), widened again."""
    return {n: t.to(BF16).float() for n, t in w.items()}


def on_device(w: dict, device, dtype) -> dict:
    """Matrices in the compute type, vectors in 32-bit, as the loader places them."""
    return {n: t.to(device, dtype if t.dim() >= 2 and not n.endswith((".conv", ".b")) else F32) for n, t in w.items()}


# =========================================================================================== each mechanism alone
@pytest.mark.parametrize("width", [40, 42, 2048])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_norm_with_a_weight_stored_around_zero(device, width, dtype):
    from ferrisinfer_b200.parts.norm import GroupedRMSNorm

    torch.manual_seed(width)
    x, w = 3.0 * torch.randn(9, width), (0.2 * torch.randn(width)).to(BF16).float()
    part = GroupedRMSNorm(width, 1e-5, weight_name="", unit_offset=True)
    assert part.tensor_specs("n")[0].name == "n"
    part.bind({"n": w.to(device)}, "n")
    out = torch.empty(9, width, dtype=dtype, device=device)
    part.forward(x.to(device), out)
    assert torch.allclose(out.cpu().double(), plain.norm_one_plus(x.double(), w.double(), 1e-5), **tol_of(dtype))
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device=device)
    out = torch.empty(3, width, dtype=dtype, device=device)
    part.forward(x.to(device), out, rows)
    assert torch.allclose(out.cpu().double(), plain.norm_one_plus(x.double(), w.double(), 1e-5)[[7, 0, 3]], **tol_of(dtype))


def gated_plain(g, u, kind, limit):
    if kind == "silu":
        return plain.silu(g) * u
    if kind == "gelu_tanh":
        return plain.gelu_tanh(g) * u
    a, b = torch.clamp(g, max=limit), torch.clamp(u, -limit, limit)
    return a * torch.sigmoid(1.702 * a) * (b + 1.0)


@pytest.mark.parametrize("kind,limit", [("silu", 0.0), ("gelu_tanh", 0.0), ("clamped_swish", 0.6), ("clamped_swish", 7.0)])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_gated_activation_kernel(device, kind, limit, dtype):
    ops = _ops()
    torch.manual_seed(3)
    gu = (2.5 * torch.randn(11, 2 * 52)).to(dtype)
    wide = torch.zeros(11, 2 * 52 + 8, dtype=dtype, device=device)  # rows further apart than they are long
    wide[:, :104] = gu.to(device)
    out = torch.empty(11, 52, dtype=dtype, device=device)
    ops.gated_activation(wide[:, :104], out, kind, limit)
    want = gated_plain(gu[:, :52].double(), gu[:, 52:].double(), kind, limit)
    assert torch.allclose(out.cpu().double(), want, **tol_of(dtype))


@pytest.mark.parametrize("kind,limit", [("gelu_tanh", 0.0), ("clamped_swish", 0.8)])
@pytest.mark.parametrize("T", [1, 8, 16, 40, 200, 700])
def test_gated_product_applies_the_activation_in_every_kernel(device, T, kind, limit):
    """bf16: the weight-stationary kernel (at most 16 tokens), the product + activation kernel in between, the
    tensor-core kernels of long steps: all against the plain gated feed-forward's inner rows; 32-bit beside them."""
    ops = _ops()
    torch.manual_seed(T)
    W, I = 128, 192
    x = torch.randn(T, W).to(BF16)
    gate_up = (torch.randn(2 * I, W) / math.sqrt(W) * 2.0).to(BF16)
    want = gated_plain(x.double() @ gate_up[:I].double().T, x.double() @ gate_up[I:].double().T, kind, limit)
    for dtype in (BF16, F32):
        out = torch.empty(T, I, dtype=dtype, device=device)
        ops.gemm_gated(x.to(device, dtype), gate_up.to(device, dtype), out, kind, limit)
        assert torch.allclose(out.cpu().double(), want, **tol_of(dtype, 2.0)), dtype


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_gate_on_rows_with_a_factor(device, dtype):
    ops = _ops()
    torch.manual_seed(5)
    x, g = torch.randn(7, 44).to(dtype), (2.0 * torch.randn(7, 44)).to(dtype)
    both = torch.cat([x, g], dim=1).to(device)
    out = torch.empty(7, 44, dtype=dtype, device=device)
    ops.gate_mul(both[:, :44], both[:, 44:], out, "sigmoid", 0.8)
    assert torch.allclose(out.cpu().double(), x.double() * torch.sigmoid(g.double()) * 0.8, **tol_of(dtype))
    ops.gate_mul(both[:, :44], both[:, 44:], both[:, :44], "silu", 1.0)  # in place
    assert torch.allclose(both[:, :44].cpu().double(), x.double() * plain.silu(g.double()), **tol_of(dtype))


def test_factor_on_the_logits(device):
    from ferrisinfer_b200.parts.embedding import OutputHead

    torch.manual_seed(6)
    table, y = torch.randn(50, 24), torch.randn(3, 24)
    head = OutputHead(50, 24, tied_to="embed", logit_scale=-2.5)
    head.bind({"embed": table.to(device)}, "head")
    logits = torch.empty(3, 50, device=device)
    head.forward(y.to(device), logits)
    assert torch.allclose(logits.cpu(), (y @ table.T) * -2.5, atol=1e-4)


def recurrent_weights(W, C, blocks, taps, seed):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    bs = C // blocks
    return rounded({
        "m.y": r(C, W) / math.sqrt(W), "m.y.b": 0.2 * r(C), "m.x": r(C, W) / math.sqrt(W), "m.x.b": 0.2 * r(C),
        "m.conv": r(C, taps) / math.sqrt(taps), "m.conv.b": 0.2 * r(C), "m.ra": 2.0 * r(blocks, bs, bs) / math.sqrt(bs),
        "m.ra.b": 0.2 * r(blocks, bs), "m.ri": 2.0 * r(blocks, bs, bs) / math.sqrt(bs), "m.ri.b": 0.2 * r(blocks, bs),
        "m.lam": -6.0 + 5.0 * torch.rand(C, generator=g), "m.o": r(W, C) / math.sqrt(C)})


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("C,blocks,taps", [(48, 3, 4), (40, 5, 1), (36, 36, 5), (72, 1, 2), (200, 2, 3)])
def test_recurrent_unit_whole_in_portions_and_token_by_token(device, C, blocks, taps, dtype):
    """The part itself (product with biases, convolution, gates, scan, output product): one request's tokens in one go
    (several tiles of the scan), in portions of unequal size and one by one from the state its slot holds, in a slot
    between slots that hold other numbers."""
    from ferrisinfer_b200.parts.base import LayerCache
    from ferrisinfer_b200.parts.recurrent import GatedLinearUnit

    W, T = 40, 300
    w = recurrent_weights(W, C, blocks, taps, C + taps)
    torch.manual_seed(C)
    y = torch.randn(T, W).to(dtype)
    want, (_, last) = plain.recurrent_unit(y.double(), {n: t.double() for n, t in w.items()}, "m",
                                           {"width": C, "blocks": blocks, "conv": taps})
    part = GatedLinearUnit(W, C, blocks, taps)
    part.bind(on_device(w, device, dtype), "m")
    for cuts in ([T], [7, 1, 130, 2, 160], [63, 1, 64, 65, 2] + [1] * 105):
        state = torch.randn(3, C, device=device)
        history = torch.randn(3, max(taps - 1, 1), C, device=device)
        state[2], history[2] = 0.0, 0.0
        need = part.cache_need()
        cache = LayerCache(need=need, parts=[None if taps == 1 else LayerCache(need=need.needs[0], state=history[:, :taps - 1].contiguous()),
                                             LayerCache(need=need.needs[1], state=state)])
        pos = 0
        for n in cuts:
            ctx = fake_ctx(device, [n], [pos], [2], act_dtype=dtype)
            h = torch.zeros(n, W, device=device)
            part.forward(y[pos:pos + n].to(device).contiguous(), h, ctx, cache, True)
            assert torch.allclose(h.cpu().double(), want[pos:pos + n], **tol_of(dtype, 5.0)), (cuts[:3], pos)
            pos += n
        if dtype == F32:
            assert torch.allclose(state[2].cpu().double(), last, atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("T,C,blocks", [(256, 64, 1), (300, 256, 2), (461, 384, 3), (1000, 128, 2)])
def test_gates_on_tensor_cores_against_the_plain_gates(device, T, C, blocks):
    """Long bf16 steps with gate blocks of a multiple of 64 channels: log a and the gated input from the tensor-core form
    (weights as stored) against the plain formulas and against the CUDA-core form (weights transposed)."""
    ops = _ops()
    torch.manual_seed(T + C)
    bs = C // blocks
    u = torch.randn(T, C).to(BF16)
    ra, ri = (2.0 * torch.randn(blocks, bs, bs) / math.sqrt(bs)).to(BF16), (2.0 * torch.randn(blocks, bs, bs) / math.sqrt(bs)).to(BF16)
    ba, bi, lam = 0.2 * torch.randn(C), 0.2 * torch.randn(C), -6.0 + 5.0 * torch.rand(C)
    rate = torch.nn.functional.softplus(lam.double()).float()
    ub = u.double().reshape(T, blocks, bs)
    r = torch.sigmoid(torch.einsum("tnk,nok->tno", ub, ra.double()).reshape(T, C) + ba.double())
    i = torch.sigmoid(torch.einsum("tnk,nok->tno", ub, ri.double()).reshape(T, C) + bi.double())
    log_a = -8.0 * r * rate.double()
    want_b = torch.sqrt(1.0 - torch.exp(2.0 * log_a)) * i * u.double()
    dev = lambda t: t.to(device)
    outs = []
    for stored in (None, (dev(ra), dev(ri))):
        a, b = torch.empty(T, C, device=device), torch.empty(T, C, device=device)
        ops.rglru_gates(dev(u), dev(ra.transpose(1, 2).contiguous()), dev(ri.transpose(1, 2).contiguous()), dev(ba), dev(bi),
                        dev(rate), a, b, 8.0, stored=stored)
        assert torch.allclose(a.cpu().double(), log_a, atol=1e-5, rtol=1e-4), stored is None
        assert torch.allclose(b.cpu().double(), want_b, atol=1e-5, rtol=1e-4), stored is None
        outs.append((a, b))
    assert ops.RGLRU_TENSOR_CORE_MIN_TOKENS <= T  # the second pass ran the tensor-core kernel


def test_scan_carries_a_write_over_hundreds_of_tokens_and_several_requests(device):
    """A decay of one (a logarithm of zero) everywhere but where a token writes: what token 3 wrote is read 700 tokens later, through tiles of
    the scan, portions that end in the middle of a tile and single tokens; three requests of unequal length in one
    step, over slots out of order, each with its own write."""
    ops = _ops()
    C = 70
    lengths, slots = [704, 130, 1], [2, 0, 3]
    T = sum(lengths)
    a = torch.zeros(T, C)  # logarithms of the decays
    b = torch.zeros(T, C)
    starts = [0, 704, 834]
    marks = {0: 3, 1: 129, 2: 0}  # the token of each request that writes
    for s, t in marks.items():
        a[starts[s] + t] = math.log(0.25)
        b[starts[s] + t] = torch.arange(C) + 10.0 * s + 1.0
    state = torch.full((5, C), 8.0, device=device)
    out = torch.empty(T, C, device=device)
    ctx = fake_ctx(device, lengths, [0, 0, 0], slots)
    ops.rglru_scan(a.to(device), b.to(device), None, out, state, ctx, gelu=False)
    for s, t in marks.items():
        wrote = 0.25 * 8.0 + torch.arange(C) + 10.0 * s + 1.0
        rows = out[starts[s]:starts[s] + lengths[s]].cpu()
        assert torch.equal(rows[:t], torch.full((t, C), 8.0))
        assert torch.allclose(rows[t:], wrote.expand(lengths[s] - t, C), rtol=1e-6, atol=0) and torch.equal(rows[t:], rows[t:t + 1].expand(lengths[s] - t, C))
        assert torch.equal(state[slots[s]].cpu(), rows[-1])
    assert torch.equal(state[1].cpu(), torch.full((C,), 8.0)) and torch.equal(state[4].cpu(), torch.full((C,), 8.0))
    # the same in portions that end inside a tile, then single tokens
    state2 = torch.full((5, C), 8.0, device=device)
    pos, rows = 0, []
    for n in [5, 64, 63, 130, 2, 400] + [1] * 40:
        ctx = fake_ctx(device, [n], [pos], [2])
        part = torch.empty(n, C, device=device)
        ops.rglru_scan(a[pos:pos + n].to(device), b[pos:pos + n].to(device), None, part, state2, ctx, gelu=False)
        rows.append(part.cpu())
        pos += n
    assert pos == 704 and torch.equal(torch.cat(rows), out[:704].cpu())


def test_a_decay_close_to_one_is_never_rounded(device):
    """Channels whose decay stays at 0.9999 to 0.999 for 4,000 tokens: what the first token wrote is left as exp(4,000 x
    log a), to 1e-5 of itself in 32-bit.  A decay formed as exp(log a) and rounded to 24 bits would be off by up to 3e-8 at
    every step with the same sign, 1e-4 of the remembered value at the end.  The scan in one portion (tiles), in portions
    and token by token; the linear attention's recurrence token after token, and as segments side by side."""
    ops = _ops()
    C, N = 96, 4000
    log_a = -torch.logspace(-4, -3, C, dtype=F64)
    want = torch.exp((N - 1) * log_a)  # the first token writes 1, the others only decay it
    a = log_a.float().expand(N, C).contiguous().to(device)
    b = torch.zeros(N, C, device=device)
    b[0] = 1.0
    exact = torch.exp((N - 1) * log_a.float().double())  # (the logarithms themselves are rounded once, to fp32)
    for cuts in ([N], [1000, 7, 2000, 993], [3900] + [1] * 100):
        state = torch.zeros(1, C, device=device)
        pos = 0
        for n in cuts:
            out = torch.empty(n, C, device=device)
            ops.rglru_scan(a[pos:pos + n], b[pos:pos + n], None, out, state, fake_ctx(device, [n], [pos], [0]), gelu=False)
            pos += n
        err = ((state[0].cpu().double() - exact) / exact).abs().max()
        assert float(err) < 2e-5, (cuts[:2], float(err))
    assert float(((exact - want) / want).abs().max()) < 1e-4  # what rounding the logarithms alone costs
    # the linear attention: rows whose decay is sigmoid(z)^(1/16) with z from 5 to 9
    d, dv = 32, 8
    z = torch.linspace(5.0, 9.0, d, dtype=F64)
    la = -torch.nn.functional.softplus(-z.float().double()) / 16.0
    exact = torch.exp((N - 1) * la)
    k = torch.zeros(N, d)
    k[0] = 1.0
    rows = torch.cat([torch.zeros(N, d), k, torch.ones(N, dv)], dim=1).to(device)
    zz = z.float().expand(N, d).contiguous().to(device)
    for segment, cuts in ((None, [250] * 16), (128, [N])):
        state = torch.zeros(1, 1, dv, d, device=device)
        pos = 0
        for n in cuts:
            r = rows[pos:pos + n]
            out = torch.empty(n, dv, device=device)
            ops.row_decay_recurrence(r[:, :d], r[:, d:2 * d], r[:, 2 * d:], zz[pos:pos + n], 1.0 / 16.0, out, state,
                                     fake_ctx(device, [n], [pos], [0]), 1, d, dv, segment=segment)
            pos += n
        err = ((state[0, 0, 3].cpu().double() - exact) / exact).abs().max()
        assert float(err) < 2e-5, (segment, float(err))


def linear_weights(W, H, d, dv, rank, seed):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    return rounded({"m.q": r(H * d, W) / math.sqrt(W), "m.k": r(H * d, W) / math.sqrt(W), "m.v": r(H * dv, W) / math.sqrt(W),
                    "m.g": r(H * dv, W) / math.sqrt(W), "m.o": r(W, H * dv) / math.sqrt(H * dv), "m.norm": 1.0 + 0.1 * r(dv),
                    "m.a1": r(rank, W) / math.sqrt(W), "m.a2": r(H * d, rank) / math.sqrt(rank), "m.a2.b": 2.0 + r(H * d)})


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("H,d,dv,rank,tau", [(2, 16, 32, 8, 8.0), (3, 8, 24, 5, 1.0), (1, 40, 8, 16, 3.0), (2, 64, 16, 3, 16.0),
                                              (1, 128, 24, 16, 16.0), (1, 136, 16, 4, 32.0), (1, 256, 40, 1, 64.0)])
def test_gated_linear_attention_whole_in_portions_and_token_by_token(device, H, d, dv, rank, tau, dtype):
    """The part itself (one product for q, k, v, the gate and the decay's inner rows, the decay's second product in
    32-bit, the recurrence with a decay per key channel, the norm per head with its SiLU gate and the mixer's factor,
    the output product), cut as the recurrent unit above."""
    from ferrisinfer_b200.parts.base import LayerCache
    from ferrisinfer_b200.parts.recurrent import GatedLinearAttention

    W, T = 40, 200
    w = linear_weights(W, H, d, dv, rank, H * d + dv)
    torch.manual_seed(d)
    y = torch.randn(T, W).to(dtype)
    want, last = plain.gated_linear_attention(y.double(), {n: t.double() for n, t in w.items()}, "m",
                                              {"heads": H, "dim": d, "vdim": dv, "tau": tau}, 1e-5)
    part = GatedLinearAttention(W, H, d, dv, tau, 1e-5, output_scale=1.3)
    assert any(n < 0 for s in part.tensor_specs("m") for n in s.shape)  # the rank is the folder's to say
    part.bind(on_device(w, device, dtype), "m")
    assert part.decay_rank == rank
    for cuts in ([T], [7, 1, 100, 2, 90], [150] + [1] * 50):
        state = torch.randn(3, H, dv, d, device=device)
        state[1] = 0.0
        cache = LayerCache(need=part.cache_need(), state=state)
        pos = 0
        for n in cuts:
            ctx = fake_ctx(device, [n], [pos], [1], act_dtype=dtype)
            h = torch.zeros(n, W, device=device)
            part.forward(y[pos:pos + n].to(device).contiguous(), h, ctx, cache, True)
            assert torch.allclose(h.cpu().double(), 1.3 * want[pos:pos + n], **tol_of(dtype, 5.0)), (cuts[:3], pos)
            pos += n
        if dtype == F32:  # S lies transposed in its slot
            assert torch.allclose(state[1].cpu().double().transpose(1, 2), last, atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("H,d,dv,segment", [(2, 16, 32, 16), (1, 40, 8, 128), (3, 64, 24, 50), (1, 136, 16, 128)])
def test_row_decay_recurrence_in_segments_side_by_side(device, H, d, dv, segment, dtype):
    """Long portions as segments side by side (sums, carry, outputs) against the same requests token after token:
    three requests of unequal length in one step, over slots out of order and from states that are not zero; one of
    them shorter than a segment, one an exact multiple."""
    ops = _ops()
    torch.manual_seed(H * d + segment)
    lengths, slots = [3 * segment, 5, 2 * segment + 7], [3, 0, 1]
    T = sum(lengths)
    q, k = (torch.randn(T, H * d) / math.sqrt(d)).to(dtype), (torch.randn(T, H * d) / math.sqrt(d)).to(dtype)
    v = torch.randn(T, H * dv).to(dtype)
    z = 2.0 + 2.0 * torch.randn(T, H * d)
    start = torch.randn(5, H, dv, d)
    rows = torch.cat([q, k, v], dim=1).to(device)
    views = (rows[:, :H * d], rows[:, H * d:2 * H * d], rows[:, 2 * H * d:])
    ctx = fake_ctx(device, lengths, [0, 0, 0], slots)
    want, want_state = torch.empty(T, H * dv, device=device), start.clone().to(device)
    ops.row_decay_recurrence(*views, z.to(device), 0.25, want, want_state, ctx, H, d, dv, q_scale=0.5)
    got, got_state = torch.empty(T, H * dv, device=device), start.clone().to(device)
    ops.row_decay_recurrence(*views, z.to(device), 0.25, got, got_state, ctx, H, d, dv, q_scale=0.5, segment=segment)
    scale = float(want.abs().max())
    assert float((got - want).abs().max()) <= 2e-5 * scale
    assert torch.allclose(got_state, want_state, atol=2e-5 * float(want_state.abs().max()))
    kept = torch.empty(T, H * dv, device=device)  # without writing the state: the slots stay as they were
    ops.row_decay_recurrence(*views, z.to(device), 0.25, kept, got_state, ctx, H, d, dv, q_scale=0.5, write_state=False,
                             segment=segment)
    assert torch.allclose(got_state, want_state, atol=2e-5 * float(want_state.abs().max()))


def test_linear_attention_reads_a_write_from_hundreds_of_tokens_ago_along_a_channel_that_does_not_decay(device):
    """Key channel 0 keeps everything (its decay is sigmoid(40)^(1/tau) = 1), the other channels forget quickly: what
    token 3 wrote along channel 0 is read 600 tokens later by a query along channel 0, while every other token writes
    along the other channels.  Portions of 200, of 64 and single tokens in between."""
    ops = _ops()
    H, d, dv, T = 1, 32, 16, 604
    torch.manual_seed(8)
    k = torch.zeros(T, d)
    k[:, 1:] = torch.randn(T, d - 1) / 4.0
    k[3] = 0.0
    k[3, 0] = 2.0
    q = torch.zeros(T, d)
    q[:, 0] = 1.0
    v = torch.randn(T, dv)
    z = torch.full((T, d), -1.0)
    z[:, 0] = 40.0
    qkv = torch.cat([q, k, v], dim=1).to(device)
    state = torch.zeros(1, H, dv, d, device=device)
    pos, outs = 0, []
    for n in [200, 200, 64, 76] + [1] * 64:
        ctx = fake_ctx(device, [n], [pos], [0])
        out = torch.empty(n, dv, device=device)
        rows = qkv[pos:pos + n]
        ops.row_decay_recurrence(rows[:, :d], rows[:, d:2 * d], rows[:, 2 * d:], z[pos:pos + n].to(device), 0.25, out, state,
                                 ctx, H, d, dv, q_scale=0.5)
        outs.append(out.cpu())
        pos += n
    got = torch.cat(outs)
    assert float(got[:3].abs().max()) == 0.0
    for t in (3, 4, 150, 400, 540, 603):
        assert torch.allclose(got[t], 0.5 * 2.0 * v[3], atol=1e-5), t


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("layout", ["interleaved", "half"])
@pytest.mark.parametrize("nh,nkv,d,dv,dims,normed", [(4, 2, 32, 48, 16, True), (3, 1, 24, 40, 24, True), (2, 2, 16, 8, 2, True),
                                                      (1, 1, 200, 16, 64, True), (9, 3, 8, 8, 0, True), (2, 1, 40, 24, 40, False)])
def test_norm_per_head_rotation_and_cache_write(device, nh, nkv, d, dv, dims, normed, layout, dtype):
    """The kernel between the q/k/v product and attention: every head divided by its own root mean square, one weight of
    ``d`` numbers for all query heads and one for all key heads, part of every head rotated, keys and values into the
    pages; from rows that are longer than q, k and v (the output gate's columns lie behind them)."""
    ops = _ops()
    torch.manual_seed(nh * d + dims)
    T, ps, eps, base = 21, 4, 1e-5, 10000.0
    rows = torch.randn(T, (nh + nkv) * d + nkv * dv + 24).to(dtype)
    wq, wk = (1.0 + 0.2 * torch.randn(d), 1.0 + 0.2 * torch.randn(d)) if normed else (None, None)
    positions = list(range(5, 5 + T))
    q = rows[:, :nh * d].double().reshape(T, nh, d)
    k = rows[:, nh * d:(nh + nkv) * d].double().reshape(T, nkv, d)
    v = rows[:, (nh + nkv) * d:(nh + nkv) * d + nkv * dv].double().reshape(T, nkv, dv)
    if normed:
        q, k = plain.norm_plain(q, wq.double(), eps), plain.norm_plain(k, wk.double(), eps)

    def rotate(x):
        if layout == "interleaved":
            return plain.rotate_pairs(x, positions, {"dims": dims, "base": base})
        out = x.clone()
        for i in range(dims // 2):
            ang = torch.tensor([p * base ** (-2.0 * i / dims) for p in positions], dtype=F64)[:, None]
            out[:, :, i] = x[:, :, i] * torch.cos(ang) - x[:, :, i + dims // 2] * torch.sin(ang)
            out[:, :, i + dims // 2] = x[:, :, i + dims // 2] * torch.cos(ang) + x[:, :, i] * torch.sin(ang)
        return out

    q, k = rotate(q), rotate(k)
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64).float().to(device)
    table = ops.RotaryTable(freq, dims, layout == "interleaved", 1.0) if dims else None
    order = [5, 0, 3, 1, 4, 2]
    kc = torch.zeros(7, nkv, ps, d, dtype=dtype, device=device)
    vc = torch.zeros(7, nkv, ps, dv, dtype=dtype, device=device)
    slots = torch.tensor([order[t // ps] * ps + t % ps for t in range(T)], dtype=torch.int32, device=device)
    ctx = fake_ctx(device, [T], [5], [0])
    dev = rows.to(device)
    view = dev[:, :(nh + nkv) * d + nkv * dv]
    ops.qk_norm_rotary_cache_write(view, ctx, slots, kc, vc, nh, nkv, d, dv, None if wq is None else wq.to(device),
                                   None if wk is None else wk.to(device), eps, table, per_head=True)
    tol = tol_of(dtype, 2.0)
    assert torch.allclose(dev[:, :nh * d].cpu().double().reshape(T, nh, d), q, **tol)
    assert torch.equal(dev[:, (nh + nkv) * d:].cpu(), rows[:, (nh + nkv) * d:])  # what lies behind is left alone
    for t in range(T):
        page, at = order[t // ps], t % ps
        assert torch.allclose(kc[page, :, at].cpu().double(), k[t], **tol), t
        assert torch.equal(vc[page, :, at].cpu().double(), v[t]), t


def attention_weights(W, H, G, d, dv, seed):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    return rounded({"m.q": r(H * d, W) / math.sqrt(W), "m.q.b": 0.2 * r(H * d), "m.k": r(G * d, W) / math.sqrt(W),
                    "m.k.b": 0.2 * r(G * d), "m.v": r(G * dv, W) / math.sqrt(W), "m.v.b": 0.2 * r(G * dv),
                    "m.q.norm": 1.0 + 0.1 * r(d), "m.k.norm": 1.0 + 0.1 * r(d), "m.g": r(H * dv, W) / math.sqrt(W),
                    "m.o": r(W, H * dv) / math.sqrt(H * dv)})


def attention_part(W, m, eps=1e-5, scale=1.0):
    from ferrisinfer_b200.parts.attention import GroupedQueryAttention
    from ferrisinfer_b200.parts.plan import PartSpec

    rot = m.get("rot")
    position = PartSpec("none") if not rot else PartSpec("scaled_rotary", {
        "rotary_dim": rot["dims"], "base": rot["base"], "layout": "interleaved", "scaling": None})
    return GroupedQueryAttention(
        W, m["heads"], m["kv_heads"], m["dim"], position, scale=m["scale"], v_head_dim=m["vdim"],
        chunk=(m.get("mask") or {}).get("size"), qk_norm={"eps": eps, "per_head": True}, fp32_weights=True,
        tensor_names={"q": "q", "k": "k", "v": "v", "o": "o"}, bias_names={"q": "q.b", "k": "k.b", "v": "v.b"},
        output_gate={"name": "g", "kind": "sigmoid"}, output_scale=scale)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("m", [cases.attention(4, 2, 32, 48, chunk=48, rot=(16, 10000.0)),
                               cases.attention(3, 1, 24, 40, chunk=21, rot=(24, 100.0), scale=0.3),
                               cases.attention(6, 6, 16, 16, chunk=16), cases.attention(2, 1, 128, 64, rot=(64, 1e6)),
                               cases.attention(8, 2, 64, 8, chunk=5, rot=(2, 50.0))])
def test_attention_mixer_against_the_plain_mixer(device, m, dtype):
    """The part itself (one product for q, k, v and the gate with their biases, the norm per head, rotation, cache write,
    chunked attention with 32-bit weights, the gate and the factor, the output product) whole, as a portion behind a
    cached prefix, and token by token, over pages out of order, against the plain mixer."""
    from ferrisinfer_b200.parts.base import LayerCache, PagedMeta

    W, T, ps = 48, 90, 16
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    w = attention_weights(W, H, G, d, dv, H * d)
    torch.manual_seed(H * d)
    y = torch.randn(T, W).to(dtype)
    want = 0.8 * plain.chunk_attention(y.double(), {n: t.double() for n, t in w.items()}, "m", m, 1e-5)[0]
    part = attention_part(W, m, scale=0.8)
    part.bind(on_device(w, device, dtype), "m")
    for cuts in ([T], [40, 17] + [1] * 33, [50] + [1] * 40):
        k, _, table, slots = paged(device, dtype, T, G, d, ps, [4, 0, 3, 1, 5, 2])
        v = torch.zeros(*k.shape[:3], dv, dtype=dtype, device=device)
        cache = LayerCache(need=part.cache_need(), group=0, k=k, v=v)
        pos = 0
        for n in cuts:
            ctx = fake_ctx(device, [n], [pos], [0], act_dtype=dtype)
            ctx.paged = {0: PagedMeta(table, slots[pos:pos + n].contiguous(), ps)}
            h = torch.zeros(n, W, device=device)
            part.forward(y[pos:pos + n].to(device).contiguous(), h, ctx, cache, True)
            assert torch.allclose(h.cpu().double(), want[pos:pos + n], **tol_of(dtype, 3.0)), (cuts[:2], pos)
            pos += n


@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("chunk,key,query", [(48, 48, 95), (48, 47, 95), (48, 0, 47), (48, 47, 48), (21, 63, 83), (21, 62, 83),
                                             (16, 240, 255), (16, 239, 255), (200, 200, 399), (200, 199, 399), (None, 1, 399),
                                             (None, 0, 16), (32, 31, 32), (32, 32, 32)])
def test_one_key_stands_out_just_inside_and_just_outside_the_chunk(device, chunk, key, query, decoded):
    """Through the whole attention mixer: queries and keys are unit directions (identity matrices, the keys shifted by
    five elements), so the score of one key is large and every other score is nothing; that key lies at the start or the
    end of the query's chunk, at a page border, hundreds of positions back, or one position outside, where it must not be
    seen.  The query comes at the end of a prompt's portion, or alone after it."""
    from ferrisinfer_b200.parts.base import LayerCache, PagedMeta

    d, ps, shift = 32, 16, 5
    m = cases.attention(1, 1, d, d, chunk=chunk, scale=0.5)
    eye = torch.eye(d)
    w = {"m.q": eye, "m.k": torch.roll(eye, shift, 0), "m.v": eye, "m.g": torch.zeros(d, d), "m.o": eye,
         "m.q.b": torch.zeros(d), "m.k.b": torch.zeros(d), "m.v.b": torch.zeros(d), "m.q.norm": torch.ones(d),
         "m.k.norm": torch.ones(d)}
    T = query + 1
    y = torch.zeros(T, d)
    y[:, 1] = 1.0  # every other token: key along element 6, value along element 1
    y[key] = 0.0
    y[key, d - shift] = 1.0  # its key lies along element 0, its value along element d - shift
    y[query] = 0.0
    y[query, 0] = 1.0  # the query along element 0; its own key along element 5, its own value along element 0
    first = 0 if chunk is None else query - query % chunk
    visible = query - first + 1  # keys of the query's chunk up to itself
    stands_out = first <= key < query  # (where the key is the query itself, its own key lies along element 5 like any other's)
    big = math.exp(0.5 * d) if stands_out else 0.0  # normed unit directions have a length of sqrt(d); every other score is 0
    total = big + (visible - (1 if stands_out else 0))
    want = torch.zeros(d, dtype=F64)
    want[d - shift] = big / total  # the value of the key that stands out
    want[0] = 1.0 / total  # the query's own value
    want[1] = (visible - 1 - (1 if stands_out else 0)) / total  # everybody else's
    want = 0.5 * want  # the gate's matrix is nothing: sigmoid(0)
    part = attention_part(d, m, eps=0.0)
    part.bind({n: t.to(device) for n, t in w.items()}, "m")
    pages = -(-T // ps)
    order = list(range(pages))
    random.Random(query).shuffle(order)
    k, _, table, slots = paged(device, F32, T, 1, d, ps, order)
    cache = LayerCache(need=part.cache_need(), group=0, k=k, v=torch.zeros_like(k))
    cuts = [T - 1, 1] if decoded and T > 1 else [T]
    pos = 0
    for n in cuts:
        ctx = fake_ctx(device, [n], [pos], [0])
        ctx.paged = {0: PagedMeta(table, slots[pos:pos + n].contiguous(), ps)}
        h = torch.zeros(n, d, device=device)
        part.forward(y[pos:pos + n].to(device).contiguous(), h, ctx, cache, True)
        pos += n
    assert torch.allclose(h[-1].cpu().double(), want, atol=1e-5), (h[-1].cpu(), want)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("T,W,E,I,top,groups", [(1, 40, 5, 0, 1, (1, 1)), (9, 44, 6, 2, 2, (4, 2)), (70, 64, 2, 3, 5, (5, 5)),
                                                 (33, 256, 60, 4, 8, (8, 3)), (5, 72, 39, 1, 20, (2, 1)), (297, 48, 4, 2, 3, (3, 2)),
                                                 (400, 72, 9, 0, 2, (3, 1))])
def test_scored_router_choices_and_weights(device, T, W, E, I, top, groups, dtype):
    """Both forms of the router kernel (a block per token, a warp per token) against the plain router: the chosen set, the
    weights in the order of the choices, identity experts handed on as one index past the last expert and their
    weights summed per token."""
    ops = _ops()
    torch.manual_seed(T + E)
    n = E + I
    router = {"experts": E, "identity": I, "top": top, "groups": {"count": groups[0], "keep": groups[1]}}
    rw = (3.0 * torch.randn(n, W) / math.sqrt(W)).to(BF16)
    corr = (0.3 * torch.randn(n) / n).to(BF16).float()
    x = torch.randn(T, W).to(dtype)
    ids = torch.empty(T, top, dtype=torch.int32, device=device)
    weights = torch.empty(T, top, device=device)
    idw = torch.full((T,), -1.0, device=device)
    ops.moe_router(x.to(device), rw.to(device, dtype), None, ids, weights, top,
                   scored={"correction": corr.to(device), "groups": groups[0], "keep": groups[1], "with_weights": E,
                           "identity_w": idw if I else None})
    w = {"m.router": rw.double(), "m.correction": corr.double()}
    checked = 0
    for t in range(T):
        chosen, wts, margin = plain.route(x[t].double(), w, "m", router)
        if margin < (1e-5 if dtype == F32 else 2e-3):
            continue  # a choice that rounding can turn
        checked += 1
        assert ids[t].tolist() == [min(e, E) for e in chosen], t
        assert torch.allclose(weights[t].cpu().double(), torch.stack(wts), **tol_of(dtype)), t
        if I:
            assert abs(float(idw[t]) - sum(float(g) for e, g in zip(chosen, wts) if e >= E)) < (1e-5 if dtype == F32 else 2e-2)
    assert checked > (T // 2 if dtype == F32 else 0) or T == 1  # (with many outputs most bfloat16 choices are close calls)


def test_scored_router_breaks_ties_by_the_lowest_index_and_leaves_groups_out_whatever_they_score(device):
    ops = _ops()
    W = 8
    rw = torch.zeros(8, W)  # every score equal: the correction decides alone
    corr = torch.tensor([0.0, 0.0, -1.0, -2.0, 0.5, -9.0, 0.5, 0.0])
    x = torch.randn(3, W)
    ids = torch.empty(3, 3, dtype=torch.int32, device=device)
    weights = torch.empty(3, 3, device=device)
    # pairs of neighbours of which all, or the two best, stay; then halves of which the better stays
    for groups, keep, want in ((4, 4, [4, 6, 0]), (4, 2, [4, 6, 7]), (2, 1, [4, 6, 7])):
        ops.moe_router(x.to(device), rw.to(device), None, ids, weights, 3,
                       scored={"correction": corr.to(device), "groups": groups, "keep": keep, "with_weights": 8})
        assert ids.tolist() == [want] * 3 and torch.allclose(weights.cpu(), torch.full((3, 3), 1.0 / 3.0))
    # negative choice scores everywhere: a group that is left out must not come back as "zero"
    ids, weights = torch.empty(3, 2, dtype=torch.int32, device=device), torch.empty(3, 2, device=device)
    ops.moe_router(x.to(device), rw.to(device), None, ids, weights, 2,
                   scored={"correction": torch.tensor([-5.0, -6.0, -1.0, -2.0, -7.0, -8.0, -3.0, -4.0]).to(device), "groups": 4,
                           "keep": 1, "with_weights": 8})
    assert ids.tolist() == [[2, 3]] * 3


@pytest.mark.parametrize("dtype,grouped", [(F32, False), (BF16, False), (BF16, True)])
@pytest.mark.parametrize("T,W,ff,E,I,top,limit", [(1, 40, 24, 5, 0, 1, 1.0), (9, 48, 40, 6, 2, 2, 0.7), (70, 64, 96, 2, 3, 5, 2.0),
                                                   (300, 128, 64, 7, 1, 3, 0.5), (40, 72, 56, 1, 2, 3, 7.0)])
def test_experts_with_a_clamped_gate_and_identity_experts(device, T, W, ff, E, I, top, limit, dtype, grouped):
    """All three ways through the experts (a block per token and expert, a block per expert for few tokens, the sorted
    tensor-core form) against the plain mixture, given the plain router's choices: the clamped gate, identity experts
    whose share is the token's own row, experts that nobody chose."""
    ops = _ops()
    if grouped and (W % 8 or ff % 8):
        pytest.skip("the sorted form takes multiples of eight")
    torch.manual_seed(T + W)
    n = E + I
    w = {"m.router": 3.0 * torch.randn(n, W) / math.sqrt(W), "m.correction": 0.3 * torch.randn(n) / n}
    for e in range(E):
        w[f"m.e{e}.gate"], w[f"m.e{e}.up"] = 2.0 * torch.randn(ff, W) / math.sqrt(W), 2.0 * torch.randn(ff, W) / math.sqrt(W)
        w[f"m.e{e}.down"] = torch.randn(W, ff) / math.sqrt(ff)
    w = rounded(w)
    x = torch.randn(T, W).to(dtype)
    mlp = cases.experts(ff, E, top, identity=I, groups=(1, 1), limit=limit)
    w64 = {k: v.double() for k, v in w.items()}
    want = plain.mixture(x.double(), w64, "m", mlp)
    ids = torch.empty(T, top, dtype=torch.int32)
    weights = torch.empty(T, top)
    idw = torch.zeros(T)
    for t in range(T):
        chosen, wts, _ = plain.route(x[t].double(), w64, "m", mlp["router"])
        ids[t] = torch.tensor([min(e, E) for e in chosen])
        weights[t] = torch.stack(wts).float()
        idw[t] = sum(float(g) for e, g in zip(chosen, wts) if e >= E)
    gate_up = torch.stack([torch.cat([w[f"m.e{e}.gate"], w[f"m.e{e}.up"]]) for e in range(E)]).to(device, dtype)
    down = torch.stack([w[f"m.e{e}.down"] for e in range(E)]).to(device, dtype)
    for accumulate in (False, True):
        h = torch.ones(T, W, device=device)
        ops.moe_experts(x.to(device), gate_up, down, ids.to(device), weights.to(device), h, None, accumulate=accumulate,
                        grouped=grouped, activation="clamped_swish", limit=limit, identity_w=idw.to(device) if I else None)
        got = h.cpu().double() - (1.0 if accumulate else 0.0)
        assert torch.allclose(got, want, **tol_of(dtype, 4.0)), (accumulate, float((got - want).abs().max()))


# ================================================================================================ whole models
MODEL_CASES = sorted(cases.CASES)
LENGTHS = {"long": (150, 11), "mid": (67, 12), "short": (23, 13), "one": (1, 14), "edge": (49, 15)}


def requests_of(case, names, lengths=LENGTHS):
    return {n: wanted(case, *lengths[n])[0] for n in names}


def rows_of(case, names, lengths=LENGTHS):
    return {n: wanted(case, *lengths[n])[1] for n in names}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", MODEL_CASES)
def test_whole_prompts(device, case, dtype):
    """Also the first tokens of a sequence: every position's logits are compared, from position 0 on."""
    runner = make_runner(cases.CASES[case], weights_of(case), dtype, device)
    names = ["long", "one", "short", "edge"]
    got = helpers.replay(runner, helpers.trace_whole(requests_of(case, names)))
    check_rows(got, rows_of(case, names), dtype, f"whole prompts {case}")
    runner.cache.check_invariants()
    assert runner.cache.num_free_slots == 4 and all(g.pool.num_used == 0 for g in runner.cache.groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", MODEL_CASES)
def test_every_layer_against_the_plain_layers(device, case, dtype):
    """The residual stream after every layer, not only the logits."""
    runner = make_runner(cases.CASES[case], weights_of(case), dtype, device, graphs=False)
    ids = wanted(case, *LENGTHS["short"])[0]
    want = []
    plain.forward(cases.folder_config(cases.CASES[case]), weights_of(case), ids, after_layer=lambda i, x: want.append(x.clone()))
    got = []
    runner.model.after_run = lambda i, h: got.append(h.detach().clone().cpu())
    helpers.replay(runner, helpers.trace_whole({"a": ids}))
    assert len(got) == len(want)
    for i, (g, w) in enumerate(zip(got, want)):
        scale = float(w.abs().max())
        assert float((g.double() - w).abs().max()) <= (1e-4 if dtype == "float32" else 6e-2) * scale, (case, i)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", MODEL_CASES)
def test_token_by_token_from_the_first_token(device, case, dtype):
    """A long decode: 150 single tokens through recorded steps, over page borders and chunk edges."""
    runner = make_runner(cases.CASES[case], weights_of(case), dtype, device)
    got = helpers.replay(runner, helpers.trace_tail_decoded(requests_of(case, ["long"]), tail=149))
    check_rows(got, rows_of(case, ["long"]), dtype, f"token by token {case}")
    assert runner.graph_replays > 100  # the decode steps were replayed from graphs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", MODEL_CASES)
def test_prompt_then_decoded_tail(device, case, dtype):
    runner = make_runner(cases.CASES[case], weights_of(case), dtype, device, graphs=False)
    names = ["long", "mid", "edge"]
    got = helpers.replay(runner, helpers.trace_tail_decoded(requests_of(case, names), tail=40))
    check_rows(got, rows_of(case, names), dtype, f"prompt then single tokens {case}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", MODEL_CASES)
@pytest.mark.parametrize("sizes", [(2,), (7, 2, 13, 3, 5, 2, 16, 4, 9, 2, 31, 6), (64, 1, 2, 17)])
def test_portions(device, case, dtype, sizes):
    runner = make_runner(cases.CASES[case], weights_of(case), dtype, device)
    names = ["long", "short"] if sizes != (2,) else ["mid"]
    got = helpers.replay(runner, helpers.trace_portions(requests_of(case, names), sizes=sizes))
    check_rows(got, rows_of(case, names), dtype, f"portions of {sizes} {case}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", MODEL_CASES)
def test_mixed_batches_over_few_pages_and_slots(device, case, dtype):
    """Seven requests, at most three live, in a pool of three state slots and just enough pages: portions of some beside
    single tokens of others, requests that sit a step out, slots and pages that are used again by the next request."""
    names = ["mid", "short", "long", "one", "edge", "mid2", "short2"]
    lengths = dict(LENGTHS, mid2=(80, 21), short2=(30, 22))
    reqs = requests_of(case, names, lengths)
    steps = helpers.trace_mixed(reqs, seed=5, max_live=3)
    pages = helpers.tokens_held(steps, round_to=16) // 16
    runner = make_runner(cases.CASES[case], weights_of(case), dtype, device, num_pages=pages, max_requests=3)
    got = helpers.replay(runner, steps)
    check_rows(got, rows_of(case, names, lengths), dtype, f"mixed batches {case}")
    runner.cache.check_invariants()
    assert runner.cache.num_free_slots == 3 and all(g.pool.num_used == 0 for g in runner.cache.groups)


def test_a_batch_gives_every_request_what_it_gets_alone(device):
    """Three unequal requests in the same steps (a portion beside single tokens) against each of them alone: 32-bit
    logits agree to rounding."""
    case = "A"
    reqs = requests_of(case, ["mid", "short", "edge"])
    together = helpers.replay(make_runner(cases.CASES[case], weights_of(case), "float32", device),
                              helpers.trace_mixed(reqs, seed=9, max_live=3))
    for name, ids in reqs.items():
        alone = helpers.replay(make_runner(cases.CASES[case], weights_of(case), "float32", device), helpers.trace_whole({name: ids}))
        for p in range(len(ids)):
            assert torch.allclose(together[(name, p)], alone[(name, p)], atol=2e-4, rtol=1e-4), (name, p)


def test_pages_of_past_chunks_come_back_while_a_request_decodes(device):
    """A pool far smaller than the request: the pages of the chunks that are over carry it on."""
    case = "A"  # chunks of 48 = three pages
    ids, want = wanted(case, *LENGTHS["long"])
    runner = make_runner(cases.CASES[case], weights_of(case), "float32", device, num_pages=5, max_requests=1)
    got = helpers.replay(runner, helpers.trace_portions({"a": ids}, sizes=(9, 1, 2, 30, 1, 1, 5)))
    check_rows(got, {"a": want}, "float32", "few pages")
    assert all(g.pool.num_used == 0 for g in runner.cache.groups)


def test_a_slot_that_is_used_again_starts_from_zero(device):
    """One state slot: the second request takes the slot (both recurrences' states and the convolution's inputs) and the
    pages the first one left, and computes what it computes alone."""
    case = "A"
    runner = make_runner(cases.CASES[case], weights_of(case), "float32", device, num_pages=10, max_requests=1)
    names = ["long", "mid"]
    got = helpers.replay(runner, helpers.trace_portions(requests_of(case, names), sizes=(40, 3, 1)))
    check_rows(got, rows_of(case, names), "float32", "a slot used again")


@pytest.mark.parametrize("case,dtype", [("A", "float32"), ("D", "float32"), ("A", "bfloat16")])
def test_a_long_prompt_and_its_decoded_tail(device, case, dtype):
    """520 tokens, the last 40 one by one: every position against the plain implementation, so that states carried
    over hundreds of tokens and several chunks are in every logit that is compared.  In bfloat16 the portion of 480
    tokens also runs the forms of long steps (the gates of the block of 64 channels on the tensor cores, the linear
    attention's segments side by side, the sorted experts)."""
    ids, want = wanted(case, 520, 77)
    runner = make_runner(cases.CASES[case], weights_of(case), dtype, device, num_pages=48)
    got = helpers.replay(runner, helpers.trace_tail_decoded({"far": ids}, tail=40))
    check_rows(got, {"far": want}, dtype, "a long prompt and its tail")


MID = cases.config([
    cases.recurrent_layer(320, 4, 4, cases.dense(384)),
    cases.parallel_layer(cases.attention(8, 2, 80, 96, chunk=160, rot=(40, 500000.0)), cases.linear(4, 48, 64, 16.0),
                         cases.experts(192, 13, 4, identity=3, groups=(4, 2), limit=1.5), scales=(0.9, 1.2)),
    cases.recurrent_layer(192, 12, 3, cases.experts(192, 13, 4, identity=3, groups=(4, 2), limit=1.5)),
    cases.parallel_layer(cases.attention(8, 2, 80, 96, chunk=160, rot=(40, 500000.0)), cases.linear(4, 48, 64, 16.0), None),
], width=256, vocab=2000, logit_scale=0.7, ranks={1: 16, 3: 32})


@functools.lru_cache(maxsize=None)
def wider_model():
    weights = cases.make_weights(MID, seed=99)
    return weights, {name: cases.safe_sequence(MID, weights, n, seed, close_call=0.008)  # sixteen outputs: scores of 0.06
                     for name, n, seed in (("far", 400, 5), ("mid", 150, 6), ("short", 70, 7))}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_wider_model_with_pages_of_64(device, dtype):
    """Sizes nearer a real model's (a width of 256, heads of 80 with values of 96, four of sixteen router outputs, a
    vocabulary of 2,000) over pages of 64: a prompt of 400 with its decoded tail, then three requests in portions beside
    single tokens over four slots and just enough pages.  The steps of more than sixteen tokens run the sorted experts
    and the tensor-core products with their gated epilogues."""
    weights, seqs = wider_model()
    runner = make_runner(MID, weights, dtype, device, num_pages=13, page_size=64)
    got = helpers.replay(runner, helpers.trace_tail_decoded({"far": seqs["far"][0]}, tail=40))
    check_rows(got, {"far": seqs["far"][1]}, dtype, "a wider model: prompt and tail")
    got = helpers.replay(runner, helpers.trace_mixed({n: ids for n, (ids, _) in seqs.items()}, seed=3))
    check_rows(got, {n: rows for n, (_, rows) in seqs.items()}, dtype, "a wider model: mixed")
    assert all(g.pool.num_used == 0 for g in runner.cache.groups)


def write_folder(tmp_path, cfg, weights) -> str:
    from ferrisinfer_b200.weights.safetensors_io import write_safetensors

    folder = str(tmp_path / "model")
    os.makedirs(folder)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cases.folder_config(cfg), f)
    write_safetensors(os.path.join(folder, "model.safetensors"), weights)
    return folder


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(device, tmp_path, dtype):
    """A folder of the design through ``Engine.generate`` (scheduler, portions, sampling on the device): every token
    is the plain implementation's greedy choice for the same prefix (or, in bfloat16, within rounding of it)."""
    from ferrisinfer_b200 import SamplingParams
    from ferrisinfer_b200.engine.engine import Engine
    from ferrisinfer_b200.engine.scheduler import SchedulerConfig

    case = "A"
    cfg, weights = cases.CASES[case], weights_of(case)
    engine = Engine(write_folder(tmp_path, cfg, weights), dtype=dtype, page_size=16, num_pages=40,
                    scheduler=SchedulerConfig(max_batch_size=4, max_prefill_chunk_tokens=32, max_prefill_batch_tokens=48,
                                              max_sequence_length=256))
    prompts = [cases.random_ids(cfg["vocab"], n, n) for n in (5, 70, 33, 1, 90, 12)]
    new = 20
    outs = engine.generate(prompts, SamplingParams.greedy(max_new_tokens=new))
    slack = 1e-4 if dtype == "float32" else 0.15
    close = 0
    for prompt, out in zip(prompts, outs):
        ids = out.generated_token_ids()
        assert len(ids) == new
        margins = []
        logits = plain.forward(cases.folder_config(cfg), weights, prompt + ids, margins=margins)[0]
        if min(margins) < (1e-5 if dtype == "float32" else cases.CLOSE_CALL):
            close += 1  # a router's choice that rounding can turn somewhere in this sequence: nothing to compare
            continue
        for i, tok in enumerate(ids):
            row = logits[len(prompt) + i - 1]
            assert row[tok] >= row.max() - slack * float(row.std()), (dtype, len(prompt), i, tok, int(row.argmax()))
    assert close < len(prompts) if dtype == "float32" else True


def test_a_random_folder_of_the_design_loads_and_generates(device, tmp_path):
    """``write_model_folder`` draws every tensor the plan asks for (the decay's inner size at its default) and the
    engine serves the folder."""
    from ferrisinfer_b200 import SamplingParams
    from ferrisinfer_b200.engine.engine import Engine
    from ferrisinfer_b200.weights.random_init import write_model_folder

    folder = write_model_folder(cases.folder_config(cases.CASE_C), 5, str(tmp_path / "random"))
    engine = Engine(folder, dtype="bfloat16", page_size=16, num_pages=16)
    outs = engine.generate([[1, 2, 3], [4]], SamplingParams.greedy(max_new_tokens=5))
    assert all(len(o.generated_token_ids()) == 5 for o in outs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_through_the_trace_runner(device, tmp_path, dtype):
    """``bin/trace_run`` as a user runs it (a subprocess fed JSON lines, four state slots, just enough pages): a folder
    of the design is chosen by its config.json, and a mixed schedule over six requests gives the plain logits."""
    from test_trace_run_gpu import run_trace

    case = "B"
    cfg, weights = cases.CASES[case], weights_of(case)
    folder = write_folder(tmp_path, cfg, weights)
    lengths = {"a": (70, 31), "b": (33, 32), "c": (101, 33), "d": (48, 34), "e": (64, 35), "f": (90, 36)}
    reqs = requests_of(case, list(lengths), lengths)
    steps = helpers.trace_mixed(reqs, seed=2)
    got = run_trace(folder, dtype, steps, tmp_path / "out", helpers.tokens_held(steps), cfg["vocab"])
    check_rows(got, rows_of(case, list(lengths), lengths), dtype, "the trace runner")


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6])
def test_random_configuration_in_every_way_of_cutting(device, seed):
    """Configurations drawn at random (sizes, head counts and groupings, rotations, chunks, experts and their groups, the
    order and number of the layers, pages of 4 to 32), replayed whole, with a decoded tail, in portions and in mixed
    batches, in both precisions against the plain implementation."""
    rng = random.Random(seed)
    cfg = cases.random_config(rng)
    weights = cases.make_weights(cfg, seed)
    page = rng.choice([4, 8, 16, 16, 32])
    lengths = [rng.randint(1, 40), rng.randint(20, 140), rng.randint(2, 70), rng.randint(60, 160), rng.randint(1, 20)]
    safe = {f"r{i}": cases.safe_sequence(cfg, weights, n, seed * 10 + i) for i, n in enumerate(lengths)}
    reqs = {rid: s[0] for rid, s in safe.items()}
    want = {rid: s[1] for rid, s in safe.items()}
    traces = {"whole": helpers.trace_whole(reqs), "tail": helpers.trace_tail_decoded(reqs),
              "portions": helpers.trace_portions(reqs), "mixed": helpers.trace_mixed(reqs, seed)}
    for dtype in ("float32", "bfloat16"):
        for kind, steps in traces.items():
            pages = helpers.tokens_held(steps, round_to=page) // page
            runner = make_runner(cfg, weights, dtype, device, num_pages=pages, max_requests=8, page_size=page)
            got = helpers.replay(runner, steps)
            runner.cache.check_invariants()
            assert all(g.pool.num_used == 0 for g in runner.cache.groups)
            check_rows(got, want, dtype, f"{cases.folder_config(cfg)} page {page} {kind}")
