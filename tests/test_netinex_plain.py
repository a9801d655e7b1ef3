"""The Netinex decoder without a GPU: its configuration and plan, what the cache manager does with a chunked need, and
a second reading of every function of the plain implementation, element by element with ``math`` alone."""

import copy
import math
import random

import pytest
import torch

import netinex_cases as cases
import plain_netinex as plain
from ferrisinfer_b200.cache.manager import CacheManager
from ferrisinfer_b200.config import resolve_config
from ferrisinfer_b200.errors import ConfigError, UnsupportedError
from ferrisinfer_b200.parts import build_model
from ferrisinfer_b200.parts.base import FixedState, PagedKV

F64 = torch.float64


@pytest.mark.parametrize("case", sorted(cases.CASES))
def test_configuration_round_trip_and_tensor_names(case):
    cfg = cases.CASES[case]
    arch, c = resolve_config(copy.deepcopy(cfg))
    assert arch.name == "Netinex" and c.to_dict() == cfg
    model = build_model(arch.plan(c))
    got = {s.name: tuple(s.shape) for s in model.tensor_specs() if s.required}
    assert got == cases.tensor_shapes(cfg)


def test_configuration_errors():
    bad = copy.deepcopy(cases.CASE_A)
    bad["layers"][0]["mixer"]["kv_heads"] = 3
    with pytest.raises(ConfigError):
        resolve_config(bad)
    bad = copy.deepcopy(cases.CASE_A)
    bad["layers"][0]["mixer"]["vdim"] = 16  # the values are the keys
    with pytest.raises(ConfigError):
        resolve_config(bad)
    bad = copy.deepcopy(cases.CASE_A)
    bad["layers"][1]["mixer"]["decay"] = [0.5]
    with pytest.raises(ConfigError):
        resolve_config(bad)
    bad = copy.deepcopy(cases.CASE_A)
    bad["layers"][1]["mlp"]["router"]["top"] = 7
    with pytest.raises(ConfigError):
        resolve_config(bad)
    bad = copy.deepcopy(cases.CASE_A)
    bad["layers"][1]["mixer"]["rot"]["dims"] = 34
    with pytest.raises(ConfigError):
        resolve_config(bad)
    bad = copy.deepcopy(cases.CASE_A)
    bad["layers"][2]["type"] = "convolution"
    with pytest.raises(UnsupportedError):
        resolve_config(bad)
    bad = copy.deepcopy(cases.CASE_A)
    bad["layers"][2]["mlp"]["kind"] = "dense"
    with pytest.raises(UnsupportedError):
        resolve_config(bad)


def test_cache_needs_by_kind_of_layer():
    arch, c = resolve_config(cases.CASE_B)
    needs = build_model(arch.plan(c)).cache_needs()
    assert needs[0] == FixedState((3, 40, 24), torch.float32)  # the state transposed: a column of S is a row
    assert needs[1] == PagedKV(1, 40, None, None, chunk=21) and needs[2] == PagedKV(2, 16, None, None, chunk=37)
    arch, c = resolve_config(cases.CASE_C)
    assert build_model(arch.plan(c)).cache_needs()[2] == PagedKV(1, 64, None, None, chunk=None)


@pytest.mark.parametrize("chunk,page", [(48, 16), (21, 16), (16, 16), (100, 8), (5, 4)])
def test_pages_of_chunks_that_are_over_go_back(chunk, page):
    """A request that walks through several chunks, in steps of changing size: every key that a token of the step may
    read has a page, and after the step no page lies wholly before the chunk of the next token."""
    mgr = CacheManager([PagedKV(2, 8, None, None, chunk=chunk)], page, 64, 2)
    mgr.admit("a")
    rng = random.Random(chunk * 100 + page)
    total = 0
    while total < 4 * chunk + 7:
        n = rng.choice([1, 1, 2, 3, chunk // 2 + 1, chunk + 3])
        before = total
        total += n
        mgr.extend("a", total)
        table = mgr.block_table("a", 0)
        for p in range(before, total):  # every token of the step and every key it reads
            for j in range(p - p % chunk, p + 1):
                if j >= before - before % chunk:
                    assert table[j // page] >= 0, (p, j)
        mgr.commit("a", total)
        table = mgr.block_table("a", 0)
        first = (total - total % chunk) // page
        assert all(b < 0 for b in table[:first]) and all(b >= 0 for b in table[first:])
        mgr.check_invariants()
    held = sum(1 for b in mgr.block_table("a", 0) if b >= 0)
    assert held <= -(-chunk // page) + 1
    mgr.release("a")
    assert mgr.groups[0].pool.num_used == 0


# ------------------------------------------------------------------ the plain implementation, read a second time
def test_dynamic_tanh_element_by_element():
    g = torch.Generator().manual_seed(1)
    x, w, b = (torch.randn(s, generator=g, dtype=F64) for s in ((3, 5), (5,), (5,)))
    got = plain.dynamic_tanh(x, w, b, torch.tensor(0.7, dtype=F64))
    for t in range(3):
        for i in range(5):
            assert abs(float(got[t, i]) - (math.tanh(0.7 * float(x[t, i])) * float(w[i]) + float(b[i]))) < 1e-12


def test_scaled_frequencies_by_hand():
    # 8 rotated elements, base 100: f = 1, 100^-0.25, 100^-0.5, 100^-0.75; original 32, fast 4, slow 1:
    # c(r) = 8 ln(32 / (2 pi r)) / (2 ln 100): c(4) = 0.2098.., c(1) = 1.4138..; lo = 0, hi = 2; ramp = 0, 0.5, 1, 1
    f, mag = plain.frequencies(cases.rotation(8, 100.0, (8.0, 32, 4.0, 1.0)))
    base = [100.0 ** (-i / 4.0) for i in range(4)]
    want = [base[0], base[1] / 8.0 * 0.5 + base[1] * 0.5, base[2] / 8.0, base[3] / 8.0]
    assert all(abs(a - b) < 1e-15 for a, b in zip(f, want))
    assert abs(mag - (0.1 * math.log(8.0) + 1.0)) < 1e-15
    f, mag = plain.frequencies(cases.rotation(8, 100.0))
    assert f == base and mag == 1.0


@pytest.mark.parametrize("layout", ["half", "interleaved"])
def test_rotation_pairs_and_passing_elements(layout):
    g = torch.Generator().manual_seed(2)
    x = torch.randn(2, 3, 10, generator=g, dtype=F64)
    rot = cases.rotation(6, 50.0)
    got = plain.rotate(x, [5, 9], rot, layout)
    assert torch.equal(got[..., 6:], x[..., 6:])  # what lies beyond the rotated elements passes
    for n, p in enumerate([5, 9]):
        for i in range(3):
            a = p * 50.0 ** (-2.0 * i / 6)
            iu, iv = (i, i + 3) if layout == "half" else (2 * i, 2 * i + 1)
            for h in range(3):
                u, v = float(x[n, h, iu]), float(x[n, h, iv])
                assert abs(float(got[n, h, iu]) - (u * math.cos(a) - v * math.sin(a))) < 1e-12
                assert abs(float(got[n, h, iv]) - (v * math.cos(a) + u * math.sin(a))) < 1e-12


def test_mixture_by_hand():
    g = torch.Generator().manual_seed(3)
    W, ff, E, top = 6, 4, 5, 2
    w = {"m.router": torch.randn(E, W, generator=g, dtype=F64), "m.router.b": torch.randn(E, generator=g, dtype=F64)}
    for e in range(E):
        w[f"m.e{e}.gate"], w[f"m.e{e}.up"] = (torch.randn(ff, W, generator=g, dtype=F64) for _ in range(2))
        w[f"m.e{e}.down"] = torch.randn(W, ff, generator=g, dtype=F64)
    y = torch.randn(3, W, generator=g, dtype=F64)
    margins = [math.inf] * 3
    got = plain.mixture(y, w, "m", {"router": {"experts": E, "top": top}}, margins)
    for t in range(3):
        z = [sum(float(w["m.router"][e, i]) * float(y[t, i]) for i in range(W)) + float(w["m.router.b"][e]) for e in range(E)]
        order = sorted(range(E), key=lambda e: -z[e])
        assert abs(margins[t] - (z[order[1]] - z[order[2]]) / (z[order[0]] - z[order[-1]])) < 1e-12
        den = sum(math.exp(z[e]) for e in order[:top])
        want = [0.0] * W
        for e in order[:top]:
            a = []
            for j in range(ff):
                gt = sum(float(w[f"m.e{e}.gate"][j, i]) * float(y[t, i]) for i in range(W))
                up = sum(float(w[f"m.e{e}.up"][j, i]) * float(y[t, i]) for i in range(W))
                a.append(gt / (1.0 + math.exp(-gt)) * up)
            for c in range(W):
                want[c] += math.exp(z[e]) / den * sum(float(w[f"m.e{e}.down"][c, j]) * a[j] for j in range(ff))
        assert all(abs(float(got[t, c]) - want[c]) < 1e-10 for c in range(W))


def test_retention_by_hand_without_rotation():
    g = torch.Generator().manual_seed(4)
    W, H, d, dv, T = 5, 2, 3, 2, 4
    mixer = {"heads": H, "dim": d, "vdim": dv, "decay": [0.5, 0.9]}
    w = {"m.q": torch.randn(H * d, W, generator=g, dtype=F64), "m.k": torch.randn(H * d, W, generator=g, dtype=F64),
         "m.v": torch.randn(H * dv, W, generator=g, dtype=F64), "m.g": torch.randn(H * dv, W, generator=g, dtype=F64),
         "m.o": torch.randn(W, H * dv, generator=g, dtype=F64)}
    y = torch.randn(T, W, generator=g, dtype=F64)
    got, _ = plain.retention(y, w, "m", mixer, 1e-5)
    q, k, v, gate = (y @ w["m." + n].T for n in "qkvg")
    for t in range(T):
        gated = []
        for h in range(H):
            o = [0.0] * dv
            for j in range(t + 1):  # the recurrence unrolled: o_t = sum_j decay^(t - j) (q_t . k_j / sqrt(d)) v_j
                dot = sum(float(q[t, h * d + i]) * float(k[j, h * d + i]) for i in range(d)) / math.sqrt(d)
                for c in range(dv):
                    o[c] += mixer["decay"][h] ** (t - j) * dot * float(v[j, h * dv + c])
            rms = math.sqrt(sum(x * x for x in o) / dv + 1e-5)
            for c in range(dv):
                z = float(gate[t, h * dv + c])
                gated.append(o[c] / rms * z / (1.0 + math.exp(-z)))
        for c in range(W):
            assert abs(float(got[t, c]) - sum(float(w["m.o"][c, i]) * gated[i] for i in range(H * dv))) < 1e-10


def test_attention_sees_its_own_chunk_only_and_its_values_are_the_projected_keys():
    g = torch.Generator().manual_seed(5)
    W, H, G, d, T, chunk = 6, 2, 1, 4, 7, 3
    mixer = {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": 0.7, "mask": {"size": chunk}}
    w = {"m.q": torch.randn(H * d, W, generator=g, dtype=F64), "m.k": torch.randn(G * d, W, generator=g, dtype=F64),
         "m.q.norm": 1.0 + 0.1 * torch.randn(H * d, generator=g, dtype=F64),
         "m.k.norm": 1.0 + 0.1 * torch.randn(G * d, generator=g, dtype=F64)}
    w["m.o"] = torch.eye(H * d, dtype=F64)  # the heads' outputs themselves
    y = torch.randn(T, W, generator=g, dtype=F64)
    got, _ = plain.chunk_attention(y, w, "m", mixer, 1e-6)
    q, k = y @ w["m.q"].T, y @ w["m.k"].T
    qn = [[float(q[t, i]) / math.sqrt(sum(float(x) ** 2 for x in q[t]) / (H * d) + 1e-6) * float(w["m.q.norm"][i])
           for i in range(H * d)] for t in range(T)]
    kn = [[float(k[t, i]) / math.sqrt(sum(float(x) ** 2 for x in k[t]) / (G * d) + 1e-6) * float(w["m.k.norm"][i])
           for i in range(G * d)] for t in range(T)]
    for t in range(T):
        seen = [j for j in range(t + 1) if j // chunk == t // chunk]
        for h in range(H):
            s = [0.7 * sum(qn[t][h * d + i] * kn[j][i] for i in range(d)) for j in seen]
            den = sum(math.exp(x) for x in s)
            for c in range(d):
                want = sum(math.exp(x) / den * float(k[j, c]) for x, j in zip(s, seen))
                assert abs(float(got[t, h * d + c]) - want) < 1e-10


@pytest.mark.parametrize("case", sorted(cases.CASES))
def test_the_plain_implementation_cut_anywhere(case):
    """Whole, in portions, and token by token from an explicit state: the same logits."""
    cfg, weights = cases.CASES[case], cases.make_weights(cases.CASES[case], 7)
    ids = cases.random_ids(cfg["vocab"], 60, 3)
    whole, _ = plain.forward(cfg, weights, ids)
    rows, state, pos = [], None, 0
    for n in (1, 7, 2, 20, 1, 1, 28):
        logits, state = plain.forward(cfg, weights, ids[pos:pos + n], start=pos, state=state)
        rows.append(logits)
        pos += n
    assert float((torch.cat(rows) - whole).abs().max()) < 1e-9


def test_a_safe_sequence_has_no_close_call():
    cfg, weights = cases.CASE_A, cases.make_weights(cases.CASE_A, 7)
    ids, rows = cases.safe_sequence(cfg, weights, 30, 1)
    margins = [math.inf] * 30
    whole, _ = plain.forward(cfg, weights, ids, margins=margins)
    assert min(margins) >= cases.CLOSE_CALL * 0.999 and float((whole - rows).abs().max()) < 1e-9
