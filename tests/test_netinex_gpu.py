"""The Netinex decoder on the GPU against the plain implementation (``plain_netinex``, float64): each kernel of its
mechanisms alone, then whole models of several small configurations driven through the step function the ways a
server drives it (whole prompts, token by token, portions down to two tokens, mixed batches over pages and state
slots that come back), and greedy generation through the engine."""

import functools
import json
import math
import os
import random
from types import SimpleNamespace

import pytest
import torch

import helpers
import netinex_cases as cases
import plain_netinex as plain

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

    arch, c = resolve_config(cfg)
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


def fake_ctx(device, q_lens, start_pos, slots, workspace=None, act_dtype=F32):
    """The device arrays of a step, as the step function lays them out."""
    from ferrisinfer_b200.engine.workspace import Workspace

    S = len(q_lens)
    q_start = [0]
    for n in q_lens:
        q_start.append(q_start[-1] + n)
    token_seq = [s for s in range(S) for _ in range(q_lens[s])]
    positions = [start_pos[s] + i for s in range(S) for i in range(q_lens[s])]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
    return SimpleNamespace(num_tokens=q_start[-1], num_seqs=S, max_q_len=max(q_lens), workspace=workspace or Workspace(device),
                           max_kv_len=max(a + b for a, b in zip(q_lens, start_pos)), act_dtype=act_dtype,
                           token_seq=i32(token_seq), positions=i32(positions), shared={}, paged={}, single_rows=None,
                           seq_q_start=i32(q_start), seq_start_pos=i32(start_pos), seq_state_slot=i32(slots))


def tol_of(dtype, loose=1.0):
    return dict(atol=2e-5 * loose, rtol=1e-4 * loose) if dtype == F32 else dict(atol=3e-2 * loose, rtol=3e-2 * loose)


# =========================================================================================== each mechanism alone
@pytest.mark.parametrize("width", [40, 42, 64, 2048])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_dynamic_tanh(device, width, dtype):
    ops = _ops()
    torch.manual_seed(width)
    x = 3.0 * torch.randn(9, width)
    w, b, alpha = 1.0 + 0.1 * torch.randn(width), 0.2 * torch.randn(width), torch.tensor([0.8])
    want = plain.dynamic_tanh(x.double(), w.double(), b.double(), alpha.double())
    out = torch.empty(9, width, dtype=dtype, device=device)
    ops.dynamic_tanh(x.to(device), w.to(device), b.to(device), alpha.to(device), out)
    assert torch.allclose(out.cpu().double(), want, **tol_of(dtype))
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device=device)
    out = torch.empty(3, width, dtype=dtype, device=device)
    ops.dynamic_tanh(x.to(device), w.to(device), b.to(device), alpha.to(device), out, rows)
    assert torch.allclose(out.cpu().double(), want[[7, 0, 3]], **tol_of(dtype))


def test_soft_cap(device):
    z = torch.linspace(-80.0, 80.0, 1001).reshape(7, 143).contiguous()
    got = z.to(device)
    _ops().softcap_(got, 12.5)
    assert torch.allclose(got.cpu().double(), 12.5 * torch.tanh(z.double() / 12.5), atol=1e-5, rtol=1e-6)


def paged(device, dtype, T, nkv, d, page_size, order, extra_pages=1):
    """Empty caches, the block table of one request whose pages lie in ``order``, and its tokens' cache slots."""
    blocks = -(-T // page_size)
    assert len(order) >= blocks
    k = torch.zeros(len(order) + extra_pages, nkv, page_size, d, dtype=dtype, device=device)
    v = torch.zeros_like(k)
    table = torch.tensor([order[:blocks]], dtype=torch.int32, device=device)
    slots = torch.tensor([order[p // page_size] * page_size + p % page_size for p in range(T)], dtype=torch.int32, device=device)
    return k, v, table, slots


@pytest.mark.parametrize("form", ["single", "tiled", "shares"])
@pytest.mark.parametrize("chunk,last", [(48, 47), (48, 48), (48, 63), (48, 95), (21, 20), (21, 21), (21, 62), (16, 255),
                                        (100, 599), (100, 600), (7, 300)])
def test_chunked_attention_one_key_stands_out_at_each_edge(device, chunk, last, form):
    """The query at position ``last`` and one key that points its way: the first key of its chunk gets (nearly) all the
    weight, and so does the last key of the chunk before when it is made the loud one, if the mask let it through:
    the output must then be the mean of the chunk's values instead, the loud key unseen.  Pages out of order, chunk
    edges on and off page borders, hundreds of keys away from position 0."""
    ops = _ops()
    from ferrisinfer_b200.engine.workspace import Workspace

    torch.manual_seed(chunk * 1000 + last)
    nh, nkv, d, ps, T = 4, 2, 32, 16, last + 1
    direction = torch.randn(d)
    direction /= direction.norm()
    first = last - last % chunk
    values = torch.randn(T, nkv, d)
    order = torch.randperm(-(-T // ps) + 2).tolist()
    q = torch.zeros(T, nh * d)
    q[last] = (3.0 * direction).repeat(nh)
    for loud in (first, first - 1):
        if loud < 0:
            continue
        keys = torch.zeros(T, nkv, d)
        keys[loud] = 10.0 * direction
        k, v, table, slots = paged(device, F32, T, nkv, d, ps, order)
        page, off = (slots // ps).long(), (slots % ps).long()
        k[page, :, off] = keys.to(device)
        v[page, :, off] = values.to(device)
        ctx = fake_ctx(device, [1], [last], [0]) if form != "tiled" else fake_ctx(device, [T], [0], [0])
        rows = q[last:].to(device) if form != "tiled" else q.to(device)
        out = torch.empty(rows.shape[0], nh * d, device=device)
        extra = dict(max_kv_len=T, workspace=Workspace(device)) if form == "shares" else {}
        ops.paged_attention_simt(rows, out, k, v, table, ctx.token_seq, ctx.positions, nh, nkv, d, 0, 1.0, v_head_dim=d,
                                 max_q_len=T if form == "tiled" else 1, chunk=chunk, **extra)
        got = out[-1].cpu().double().view(nh, d)
        of = torch.arange(nh) // (nh // nkv)
        if loud == first:  # seen: exp(30) against exp(0) of the others
            want = values[first].double()[of]
        else:  # one position too early: every key of the chunk scores 0
            want = values[first:last + 1].double().mean(dim=0)[of]
        assert torch.allclose(got, want, atol=1e-4, rtol=1e-4), (loud - first, got[0, :3], want[0, :3])


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("layout", ["interleaved", "half"])
@pytest.mark.parametrize("nh,nkv,d,dims,normed,from_keys", [(4, 2, 32, 32, True, True), (3, 1, 40, 24, True, True),
                                                             (2, 2, 15, 6, True, True), (5, 5, 9, 8, False, False),
                                                             (16, 4, 128, 128, True, True), (2, 1, 64, 0, True, False),
                                                             (1, 1, 6, 2, False, True)])
def test_norm_over_the_projection_rotation_and_cache_write(device, nh, nkv, d, dims, normed, from_keys, layout, dtype):
    """The kernel between the q/k product and attention alone, in its paired form (even head sizes) and its general one
    (odd ones), both pair layouts, part of a head rotating, with and without the norm, values taken from the keys or
    from a third part of the row: the queries left in the row, the keys and values found in their cache slots."""
    ops = _ops()
    torch.manual_seed(nh * 100 + d)
    T, ps, eps = 37, 16, 1e-5
    rot = cases.rotation(dims, 700.0, (4.0, 64, 8.0, 2.0)) if dims else None
    f, mag = plain.frequencies(rot)
    width = (nh + nkv) * d + (0 if from_keys else nkv * d)
    rows = torch.randn(T, width).to(dtype)
    qw, kw = 1.0 + 0.2 * torch.randn(nh * d), 1.0 + 0.2 * torch.randn(nkv * d)
    positions = [3 + 5 * t for t in range(T)]
    x = rows.double()
    q, k = x[:, :nh * d], x[:, nh * d:(nh + nkv) * d]
    values = k if from_keys else x[:, (nh + nkv) * d:]
    if normed:
        q = q / torch.sqrt(q.pow(2).mean(-1, keepdim=True) + eps) * qw.double()
        k = k / torch.sqrt(k.pow(2).mean(-1, keepdim=True) + eps) * kw.double()
    q = plain.rotate(q.view(T, nh, d), positions, rot, layout).reshape(T, nh * d)
    k = plain.rotate(k.view(T, nkv, d), positions, rot, layout).reshape(T, nkv * d)
    kc, vc, _, slots = paged(device, dtype, T, nkv, d, ps, [2, 0, 1])
    ctx = SimpleNamespace(positions=torch.tensor(positions, dtype=torch.int32, device=device))
    table = None if not dims else ops.RotaryTable(torch.tensor(f, dtype=F32, device=device), dims, layout == "interleaved", mag)
    dev_rows = rows.to(device)
    ops.qk_norm_rotary_cache_write(dev_rows, ctx, slots, kc, vc, nh, nkv, d, d, qw.to(device) if normed else None,
                                   kw.to(device) if normed else None, eps, table, values_from_keys=from_keys)
    tol = tol_of(dtype)
    assert torch.allclose(dev_rows[:, :nh * d].cpu().double(), q, **tol)
    slot = slots.cpu().long()
    got_k = kc.cpu().double().permute(0, 2, 1, 3).reshape(-1, nkv * d)[slot]
    got_v = vc.cpu().double().permute(0, 2, 1, 3).reshape(-1, nkv * d)[slot]
    assert torch.allclose(got_k, k, **tol)
    assert torch.equal(got_v, values)
    # without a cache to write, the queries alone change
    again = rows.to(device)
    ops.qk_norm_rotary_cache_write(again, ctx, None, None, None, nh, nkv, d, d, qw.to(device) if normed else None,
                                   kw.to(device) if normed else None, eps, table, values_from_keys=from_keys, write_kv=False)
    assert torch.equal(again[:, :nh * d], dev_rows[:, :nh * d]) and torch.equal(again[:, nh * d:].cpu(), rows[:, nh * d:])


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("nh,nkv,d,rot,chunk", [(4, 2, 32, cases.rotation(32, 10000.0, (4.0, 64, 8.0, 2.0)), 48),
                                                  (3, 1, 40, cases.rotation(24, 100.0), 21),
                                                  (6, 6, 16, None, 16), (2, 1, 128, cases.rotation(128, 1e6, (2.0, 32, 4.0, 1.0)), None),
                                                  (8, 2, 64, cases.rotation(2, 50.0), 5)])
def test_attention_mixer_against_the_plain_mixer(device, nh, nkv, d, rot, chunk, dtype):
    """The part itself (product, norm over the whole projection, rotation, cache write, chunked attention, output
    product) whole, as a portion behind a cached prefix, and token by token (alone and in shares), over pages out of
    order, against the plain mixer."""
    from ferrisinfer_b200.parts.attention import GroupedQueryAttention
    from ferrisinfer_b200.parts.base import LayerCache, PagedMeta
    from ferrisinfer_b200.parts.plan import PartSpec

    torch.manual_seed(nh * d)
    W, T, ps = 48, 90, 16
    mixer = {"heads": nh, "kv_heads": nkv, "dim": d, "vdim": d, "scale": 2.0 / math.sqrt(d)}
    if chunk:
        mixer["mask"] = {"size": chunk}
    if rot:
        mixer["rot"] = rot
    w = {"m.q": torch.randn(nh * d, W) / math.sqrt(W), "m.k": torch.randn(nkv * d, W) / math.sqrt(W),
         "m.q.norm": 1.0 + 0.1 * torch.randn(nh * d), "m.k.norm": 1.0 + 0.1 * torch.randn(nkv * d),
         "m.o": torch.randn(W, nh * d) / math.sqrt(nh * d)}
    w = {n: t.to(BF16).float() for n, t in w.items()}
    y = torch.randn(T, W).to(dtype)
    want = plain.chunk_attention(y.double(), {n: t.double() for n, t in w.items()}, "m", mixer, 1e-5)[0]
    position = PartSpec("none") if not rot else PartSpec("scaled_rotary", {
        "rotary_dim": rot["dims"], "base": rot["base"], "layout": "interleaved", "scaling": rot.get("scaling")})
    part = GroupedQueryAttention(W, nh, nkv, d, position, scale=mixer["scale"], chunk=chunk, values_from_keys=True,
                                 qk_norm={"eps": 1e-5}, fp32_weights=True, tensor_names={"q": "q", "k": "k", "o": "o"})
    part.bind({n: t.to(device, dtype if t.dim() == 2 else F32) for n, t in w.items()}, "m")
    for cuts in ([T], [40, 17] + [1] * 33, [50] + [1] * 40):
        k, v, table, slots = paged(device, dtype, T, nkv, d, ps, [4, 0, 3, 1, 5, 2])
        cache = LayerCache(need=part.cache_need(), group=0, k=k, v=v)
        pos = 0
        for n in cuts:
            ctx = fake_ctx(device, [n], [pos], [0], act_dtype=dtype)
            ctx.paged = {0: PagedMeta(table, slots[pos:pos + n].contiguous(), ps)}
            h = torch.zeros(n, W, device=device)
            part.forward(y[pos:pos + n].to(device).contiguous(), h, ctx, cache, True)
            assert torch.allclose(h.cpu().double(), want[pos:pos + n], **tol_of(dtype, 3.0)), (cuts[:2], pos)
            pos += n


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("heads,dim,vdim,rot", [(2, 32, 32, cases.rotation(32)), (3, 24, 40, cases.rotation(16, 500.0)),
                                                 (4, 16, 16, None), (1, 128, 72, cases.rotation(128, 1e6, (2.0, 16, 4.0, 0.5))),
                                                 (2, 200, 8, cases.rotation(6, 50.0))])
def test_retention_mixer_whole_in_portions_and_token_by_token(device, heads, dim, vdim, rot, dtype):
    """The part itself (product, rotation and key factor on the way into the recurrence, per-head norm, SiLU gate, output
    product): one request's tokens in one go (long enough to run as segments side by side), in portions of unequal
    size and one by one from the state its slot holds."""
    from ferrisinfer_b200.parts.base import LayerCache
    from ferrisinfer_b200.parts.linear_attention import DecayedLinearAttention
    from ferrisinfer_b200.parts.plan import PartSpec

    torch.manual_seed(heads * dim + vdim)
    W, T = 40, 300
    decay = [1.0, 0.97, 0.5, 0.9][:heads]
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}
    if rot:
        mixer["rot"] = rot
    w = {"m.q": torch.randn(heads * dim, W) / math.sqrt(W), "m.k": torch.randn(heads * dim, W) / math.sqrt(W),
         "m.v": torch.randn(heads * vdim, W) / math.sqrt(W), "m.g": torch.randn(heads * vdim, W) / math.sqrt(W),
         "m.o": torch.randn(W, heads * vdim) / math.sqrt(heads * vdim)}
    w = {n: t.to(BF16).float() for n, t in w.items()}
    y = torch.randn(T, W).to(dtype)
    want, last = plain.retention(y.double(), {n: t.double() for n, t in w.items()}, "m", mixer, 1e-5)
    position = None if not rot else PartSpec("scaled_rotary", {
        "rotary_dim": rot["dims"], "base": rot["base"], "layout": "half", "scaling": rot.get("scaling")})
    part = DecayedLinearAttention(W, heads, dim, vdim, decay, 1e-5, activation="none", position=position,
                                  k_scale=dim ** -0.5, head_norm=True, gate="silu")
    part.bind({n: t.to(device, dtype) for n, t in w.items()}, "m")
    for cuts in ([T], [7, 1, 130, 2, 160], [260] + [1] * 40):
        state = torch.randn(3, heads, vdim, dim, device=device)
        state[2] = 0.0
        cache = LayerCache(need=part.cache_need(), state=state)
        pos = 0
        for n in cuts:
            ctx = fake_ctx(device, [n], [pos], [2], act_dtype=dtype)
            h = torch.zeros(n, W, device=device)
            part.forward(y[pos:pos + n].to(device).contiguous(), h, ctx, cache, True)
            assert torch.allclose(h.cpu().double(), want[pos:pos + n], **tol_of(dtype, 5.0)), (cuts[:3], pos)
            pos += n
        if dtype == F32:  # S lies transposed in its slot
            assert torch.allclose(state[2].cpu().double().transpose(1, 2), last, atol=1e-3, rtol=1e-3)


def test_retention_reads_a_write_from_hundreds_of_tokens_ago_through_the_rotation(device):
    """A decay of one: what token 3 wrote along one pair of rotated elements is read 700 tokens later by a query along
    the same pair, turned by the angle that 700 positions make; every other key lies along other elements.  Portions of
    200 (segments side by side), of 64, and single tokens in between."""
    ops = _ops()
    heads, dim, vdim, T = 1, 64, 32, 704
    f = 0.01  # the frequency of the pair (0, 32)
    freq = torch.zeros(dim // 2)
    freq[0] = f
    table = ops.RotaryTable(freq.to(device), dim, False, 1.0)
    k = torch.zeros(T, dim)
    k[:, 1:32] = torch.randn(T, 31) / 8.0
    k[3, :] = 0.0
    k[3, 0] = 1.0
    v = torch.randn(T, vdim)
    q = torch.zeros(T, dim)
    q[:, 0] = 1.0
    qkv = torch.cat([q, k, v], dim=1).to(device)
    state = torch.zeros(1, heads, vdim, dim, device=device)
    decay = torch.ones(1, device=device)
    pos, outs = 0, []
    for n in [200, 200, 64, 64, 112] + [1] * 64:
        ctx = fake_ctx(device, [n], [pos], [0])
        out = torch.empty(n, vdim, device=device)
        ops.linear_attention(qkv[pos:pos + n].contiguous(), (0, dim, 2 * dim), out, state, decay, ctx, heads, dim, vdim,
                             rotary=table, k_scale=0.5)
        outs.append(out.cpu())
        pos += n
    got = torch.cat(outs).double()
    for t in (3, 4, 150, 400, 640, 703):  # rotated q_t . rotated k_3 = cos((t - 3) f); only token 3 wrote along this pair
        assert float((got[t] - 0.5 * math.cos((t - 3) * f) * v[3].double()).abs().max()) < 2e-4, t


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("T,W,E,top", [(1, 40, 5, 1), (9, 44, 12, 3), (70, 64, 3, 3), (33, 256, 64, 8), (5, 72, 40, 32),
                                        (297, 48, 6, 6), (400, 72, 9, 2)])
def test_router_choices_and_weights(device, T, W, E, top, dtype):
    ops = _ops()
    torch.manual_seed(T * E)
    x = torch.randn(T, W).to(dtype)
    wr = (3.0 * torch.randn(E, W) / math.sqrt(W)).to(dtype)
    b = torch.randn(E)
    z = x.double() @ wr.double().T + b.double()
    ids = torch.empty(T, top, dtype=torch.int32, device=device)
    weights = torch.empty(T, top, device=device)
    ops.moe_router(x.to(device), wr.to(device), b.to(device), ids, weights, top)
    order = torch.argsort(z, dim=-1, descending=True, stable=True)[:, :top]
    assert torch.equal(ids.cpu().long(), order)
    want = torch.softmax(torch.gather(z, 1, order), dim=-1)
    assert torch.allclose(weights.cpu().double(), want, atol=1e-5, rtol=1e-4)
    # a token alone (a block per token) and among hundreds (a warp per token): the same bits
    ids1 = torch.empty(1, top, dtype=torch.int32, device=device)
    weights1 = torch.empty(1, top, device=device)
    ops.moe_router(x[T - 1:].to(device), wr.to(device), b.to(device), ids1, weights1, top)
    assert torch.equal(ids1[0], ids[T - 1]) and torch.equal(weights1[0], weights[T - 1])


def test_router_takes_the_lowest_index_among_equals(device):
    x = torch.zeros(2, 16, device=device)  # every logit is its bias
    b = torch.tensor([0.5, 2.0, 2.0, -1.0, 2.0, 0.5], device=device)
    ids = torch.empty(2, 4, dtype=torch.int32, device=device)
    weights = torch.empty(2, 4, device=device)
    _ops().moe_router(x, torch.zeros(6, 16, device=device), b, ids, weights, 4)
    assert ids.cpu().tolist() == [[1, 2, 4, 0]] * 2


@pytest.mark.parametrize("dtype,grouped", [(F32, False), (BF16, False), (BF16, True)])
@pytest.mark.parametrize("T,W,ff,E,top", [(1, 40, 24, 5, 1), (9, 44, 36, 12, 3), (70, 64, 96, 3, 3), (300, 128, 64, 8, 2),
                                           (17, 256, 200, 6, 4), (700, 256, 384, 16, 4), (130, 64, 72, 40, 1)])
def test_experts_against_the_plain_mixture(device, T, W, ff, E, top, dtype, grouped):
    """Router and experts together through the part, adding into the residual rows and replacing them; token by token
    (a block per token and expert) and sorted by expert (tensor-core tiles that each meet their own expert's weights:
    experts without a token, with a few, with several tiles of them)."""
    from ferrisinfer_b200.kernels import ops
    from ferrisinfer_b200.parts.feed_forward import MixtureOfExperts

    if grouped and (W % 8 or ff % 8):
        pytest.skip("rows of no multiple of 8 elements go token by token")
    was = ops.MOE_GROUPED_MIN_TOKENS
    ops.MOE_GROUPED_MIN_TOKENS = 1 if grouped else 1 << 30
    try:
        _experts_against_the_plain_mixture(device, T, W, ff, E, top, dtype)
    finally:
        ops.MOE_GROUPED_MIN_TOKENS = was


def _experts_against_the_plain_mixture(device, T, W, ff, E, top, dtype):
    from ferrisinfer_b200.parts.feed_forward import MixtureOfExperts

    torch.manual_seed(T + W)
    w = {"m.router": 3.0 * torch.randn(E, W) / math.sqrt(W), "m.router.b": torch.randn(E)}
    for e in range(E):
        w[f"m.e{e}.gate"], w[f"m.e{e}.up"] = torch.randn(ff, W) / math.sqrt(W), torch.randn(ff, W) / math.sqrt(W)
        w[f"m.e{e}.down"] = torch.randn(W, ff) / math.sqrt(ff)
    w = {n: t.to(BF16).float() for n, t in w.items()}
    y = torch.randn(T, W).to(dtype)
    margins = [math.inf] * T
    want = plain.mixture(y.double(), {n: t.double() for n, t in w.items()}, "m", {"router": {"experts": E, "top": top}}, margins)
    part = MixtureOfExperts(W, ff, E, top)
    part.bind({n: t.to(device, dtype if t.dim() == 2 else F32) for n, t in w.items()}, "m")
    ctx = fake_ctx(device, [T], [0], [0], act_dtype=dtype)
    before = torch.randn(T, W)
    h = before.to(device)
    part.forward(y.to(device), h, ctx)
    sure = torch.tensor([m > 1e-3 for m in margins])  # a choice that a rounding of the sums could turn is not compared
    assert sure.sum() >= T * 0.9
    assert torch.allclose((h.cpu().double() - before.double())[sure], want[sure], **tol_of(dtype, 3.0))
    part.forward(y.to(device), h, ctx, accumulate=False)
    assert torch.allclose(h.cpu().double()[sure], want[sure], **tol_of(dtype, 3.0))


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("W,ff", [(64, 96), (44, 36)])
def test_experts_give_a_token_the_same_bits_alone_and_among_others(device, W, ff, dtype):
    """One choice per token: a token alone goes through the kernels of a block per (token, expert), eleven tokens through
    those that read an expert's weights once for all its tokens (four at a time, so some experts take several turns)."""
    ops = _ops()
    torch.manual_seed(W)
    E, T = 3, 11
    gate_up = (torch.randn(E, 2 * ff, W) / math.sqrt(W)).to(device, dtype)
    down = (torch.randn(E, W, ff) / math.sqrt(ff)).to(device, dtype)
    x = torch.randn(T, W).to(device, dtype)
    ids = torch.tensor([[t % 2 * 2] for t in range(T)], dtype=torch.int32, device=device)  # expert 1 stays without a token
    weights = torch.rand(T, 1, device=device) + 0.5
    together = torch.zeros(T, W, device=device)
    ops.moe_experts(x, gate_up, down, ids, weights, together, None, accumulate=False, grouped=False)
    for t in range(T):
        alone = torch.zeros(1, W, device=device)
        ops.moe_experts(x[t:t + 1], gate_up, down, ids[t:t + 1], weights[t:t + 1], alone, None, accumulate=False, grouped=False)
        assert torch.equal(alone[0], together[t]), t


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
    plain.forward(cases.CASES[case], weights_of(case), ids, after_layer=lambda i, x: want.append(x.clone()))
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


def test_pages_of_past_chunks_come_back_while_a_request_decodes(device):
    """A pool far smaller than the request: the pages of the chunks that are over carry it on."""
    case = "A"  # chunks of 48 = three pages
    ids, want = wanted(case, *LENGTHS["long"])
    runner = make_runner(cases.CASES[case], weights_of(case), "float32", device, num_pages=5, max_requests=1)
    got = helpers.replay(runner, helpers.trace_portions({"a": ids}, sizes=(9, 1, 2, 30, 1, 1, 5)))
    check_rows(got, {"a": want}, "float32", "few pages")
    assert all(g.pool.num_used == 0 for g in runner.cache.groups)


def test_a_slot_that_is_used_again_starts_from_zero(device):
    """One state slot: the second request takes the slot (retention states) and the pages the first one left, and
    computes what it computes alone."""
    case = "A"
    runner = make_runner(cases.CASES[case], weights_of(case), "float32", device, num_pages=10, max_requests=1)
    names = ["long", "mid"]
    got = helpers.replay(runner, helpers.trace_portions(requests_of(case, names), sizes=(40, 3, 1)))
    check_rows(got, rows_of(case, names), "float32", "a slot used again")


def test_a_long_prompt_and_its_decoded_tail(device):
    """520 tokens, the last 40 one by one, in 32-bit: every position against the plain implementation, so that writes
    from hundreds of tokens ago (a decay of one) and several chunks are in every logit that is compared."""
    case = "C"
    ids, want = wanted(case, 520, 77)
    runner = make_runner(cases.CASES[case], weights_of(case), "float32", device, num_pages=48)
    got = helpers.replay(runner, helpers.trace_tail_decoded({"far": ids}, tail=40))
    check_rows(got, {"far": want}, "float32", "a long prompt and its tail")


MID = cases.config([cases.retention_layer(8, 32, 64, cases.experts(192, 16, 4), rot=cases.rotation(32, 500000.0), seed=7),
                    cases.attention_layer(8, 2, 80, 160, cases.experts(192, 16, 4),
                                          rot=cases.rotation(80, 10000.0, (4.0, 1024, 32.0, 1.0))),
                    cases.retention_layer(8, 32, 64, None, rot=cases.rotation(32, 500000.0), seed=8),
                    cases.attention_layer(8, 2, 80, 160, cases.experts(192, 16, 4),
                                          rot=cases.rotation(80, 10000.0, (4.0, 1024, 32.0, 1.0)))],
                   width=256, vocab=2000, softcap=20.0)


@functools.lru_cache(maxsize=None)
def wider_model():
    weights = cases.make_weights(MID, seed=99)
    return weights, {name: cases.safe_sequence(MID, weights, n, seed)
                     for name, n, seed in (("far", 400, 5), ("mid", 150, 6), ("short", 70, 7))}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_wider_model_with_pages_of_64(device, dtype):
    """Sizes nearer a real model's (a width of 256, heads of 80, four of sixteen experts, a vocabulary of 2,000) over
    pages of 64: a prompt of 400 with its decoded tail, then three requests in portions beside single tokens over four
    slots and just enough pages."""
    weights, seqs = wider_model()
    runner = make_runner(MID, weights, dtype, device, num_pages=13, page_size=64)
    got = helpers.replay(runner, helpers.trace_tail_decoded({"far": seqs["far"][0]}, tail=40))
    check_rows(got, {"far": seqs["far"][1]}, dtype, "a wider model: prompt and tail")
    got = helpers.replay(runner, helpers.trace_mixed({n: ids for n, (ids, _) in seqs.items()}, seed=3))
    check_rows(got, {n: rows for n, (_, rows) in seqs.items()}, dtype, "a wider model: mixed")
    assert all(g.pool.num_used == 0 for g in runner.cache.groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(device, tmp_path, dtype):
    """A folder of the design through ``Engine.generate`` (scheduler, portions, sampling on the device): every token
    is the plain implementation's greedy choice for the same prefix (or, in bfloat16, within rounding of it)."""
    from ferrisinfer_b200 import SamplingParams
    from ferrisinfer_b200.engine.engine import Engine
    from ferrisinfer_b200.engine.scheduler import SchedulerConfig
    from ferrisinfer_b200.weights.safetensors_io import write_safetensors

    case = "A"
    cfg, weights = cases.CASES[case], weights_of(case)
    folder = str(tmp_path / "model")
    os.makedirs(folder)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), weights)
    engine = Engine(folder, dtype=dtype, page_size=16, num_pages=40,
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
        margins = [math.inf] * (len(prompt) + new)
        logits = plain.forward(cfg, weights, prompt + ids, margins=margins)[0]
        if min(margins) < (1e-4 if dtype == "float32" else cases.CLOSE_CALL):
            close += 1  # a router's choice that rounding can turn somewhere in this sequence: nothing to compare
            continue
        for i, tok in enumerate(ids):
            row = logits[len(prompt) + i - 1]
            assert row[tok] >= row.max() - slack * float(row.std()), (dtype, len(prompt), i, tok, int(row.argmax()))
    assert close < len(prompts) if dtype == "float32" else True


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_through_the_trace_runner(device, tmp_path, dtype):
    """``bin/trace_run`` as a user runs it (a subprocess fed JSON lines, four state slots, just enough pages): a folder
    of the design is chosen by its config.json, and a mixed schedule over six requests gives the plain logits."""
    from test_trace_run_gpu import run_trace
    from ferrisinfer_b200.weights.safetensors_io import write_safetensors

    case = "B"
    cfg, weights = cases.CASES[case], weights_of(case)
    folder = str(tmp_path / "model")
    os.makedirs(folder)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), weights)
    lengths = {"a": (70, 31), "b": (33, 32), "c": (101, 33), "d": (48, 34), "e": (64, 35), "f": (90, 36)}
    reqs = requests_of(case, list(lengths), lengths)
    steps = helpers.trace_mixed(reqs, seed=2)
    got = run_trace(folder, dtype, steps, tmp_path / "out", helpers.tokens_held(steps), cfg["vocab"])
    check_rows(got, rows_of(case, list(lengths), lengths), dtype, "the trace runner")


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6])
def test_random_configuration_in_every_way_of_cutting(device, seed):
    """Configurations drawn at random (sizes, head counts and groupings, rotations, chunks, experts, the order and number
    of the layers, pages of 4 to 32), replayed whole, with a decoded tail, in portions and in mixed batches, in both
    precisions against the plain implementation."""
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
            check_rows(got, want, dtype, f"{cfg} page {page} {kind}")
