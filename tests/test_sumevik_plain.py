"""The Sumevik decoder without a GPU: its configuration and plan, what its layers ask of the cache manager, and a
second reading of every function of the plain implementation, element by element with ``math`` alone."""

import copy
import math
import random

import pytest
import torch

import plain_sumevik as plain
import sumevik_cases as cases
from ferrisinfer_b200.config import resolve_config
from ferrisinfer_b200.errors import ConfigError, UnsupportedError
from ferrisinfer_b200.parts import build_model
from ferrisinfer_b200.parts.base import FixedState, PagedKV, leaf_needs
from ferrisinfer_b200.weights.loader import check_tensors, shape_fits

F64 = torch.float64


@pytest.mark.parametrize("case", sorted(cases.CASES))
def test_configuration_round_trip_and_tensor_names(case):
    cfg = cases.folder_config(cases.CASES[case])
    arch, c = resolve_config(copy.deepcopy(cfg))
    assert arch.name == "Sumevik"
    again = c.to_dict()
    assert resolve_config(again)[1] == c  # what the typed configuration writes, it reads back as itself
    for key in ("vocab", "width", "norm"):
        assert again[key] == cfg[key]
    assert again["layers"] == cfg["layers"] and again["logit_scale"] == cfg.get("logit_scale", 1.0)
    model = build_model(arch.plan(c))
    specs = [s for s in model.tensor_specs() if s.required]
    shapes = cases.tensor_shapes(cases.CASES[case])
    assert {s.name for s in specs} == set(shapes)
    # the inner size of the decay's projection is the folder's to decide: every other size is the configuration's
    free = {s.name for s in specs if any(n < 0 for n in s.shape)}
    assert free == {n for n in shapes if n.endswith((".a1", ".a2"))}
    assert all(shape_fits(s.shape, shapes[s.name]) for s in specs)
    check_tensors(specs, shapes)


def test_a_size_that_the_folder_decides_still_has_to_fit_the_rest():
    assert shape_fits((-16, 40), (3, 40)) and shape_fits((8, -16), (8, 1))
    assert not shape_fits((-16, 40), (3, 41)) and not shape_fits((-16, 40), (40,))


def test_configuration_errors():
    def broken(change):
        bad = copy.deepcopy(cases.folder_config(cases.CASE_A))
        change(bad)
        return bad

    def set_(path, value):
        def change(d):
            for k in path[:-1]:
                d = d[k]
            d[path[-1]] = value
        return change

    for change in (set_(("layers", 0, "mixer", "blocks"), 5),  # 48 channels in 5 blocks
                   set_(("layers", 0, "mixer", "conv"), 0),
                   set_(("layers", 1, "mixer", "left", "kv_heads"), 3),
                   set_(("layers", 1, "mixer", "left", "rot", "dims"), 34),
                   set_(("layers", 1, "mixer", "left", "rot", "dims"), 7),
                   set_(("layers", 1, "mixer", "left", "mask", "size"), 0),
                   set_(("layers", 1, "mixer", "right", "tau"), 0.0),
                   set_(("layers", 1, "mlp", "router", "top"), 5),  # two groups of two stay: four at most
                   set_(("layers", 1, "mlp", "router", "groups", "count"), 3),  # eight outputs in three groups
                   set_(("layers", 1, "mlp", "router", "groups", "keep"), 5),
                   set_(("layers", 1, "mlp", "expert", "limit"), -1.0),
                   set_(("width",), 0)):
        with pytest.raises(ConfigError):
            resolve_config(broken(change))
    for change in (set_(("layers", 2, "type"), "convolution"), set_(("layers", 0, "mlp", "kind"), "sparse")):
        with pytest.raises(UnsupportedError):
            resolve_config(broken(change))


def test_what_the_configuration_leaves_out():
    """No rotation, no chunk, no groups, no identity experts, no factors: the keys are simply absent."""
    cfg = cases.folder_config(cases.config([
        cases.parallel_layer({"heads": 2, "dim": 8, "scale": 0.5}, {"heads": 1, "dim": 8, "tau": 2.0},
                             {"kind": "moe", "expert": {"ff": 8, "limit": 1.0}, "router": {"experts": 3, "top": 2}}),
    ], width=16, vocab=11))
    del cfg["layers"][0]["mixer"]["left_scale"], cfg["layers"][0]["mixer"]["right_scale"]
    arch, c = resolve_config(cfg)
    layer = c.layers[0]
    a, g, e = layer.mixer.left, layer.mixer.right, layer.mlp
    assert (a.kv_heads, a.vdim, a.chunk, a.rot_dims) == (2, 8, None, 0) and g.vdim == 8
    assert (layer.mixer.left_scale, layer.mixer.right_scale, c.logit_scale) == (1.0, 1.0, 1.0)
    assert (e.identity, e.group_count, e.group_keep) == (0, 1, 1)
    build_model(arch.plan(c))


def test_cache_needs_by_kind_of_layer():
    arch, c = resolve_config(cases.folder_config(cases.CASE_A))
    needs = build_model(arch.plan(c)).cache_needs()
    first = leaf_needs(needs[0])  # the recurrent unit: the convolution's last three inputs and the state, one row each
    assert [type(n) for n in first] == [FixedState, FixedState]
    assert first[0].shape == (3, 48) and first[1].shape == (48,) and first[1].dtype == torch.float32
    second = leaf_needs(needs[1])  # side by side: pages of a chunk for the left, a state for the right
    assert isinstance(second[0], PagedKV) and isinstance(second[1], FixedState)
    assert (second[0].num_kv_heads, second[0].head_dim, second[0].value_dim, second[0].chunk) == (2, 32, 48, 48)
    assert second[0].first_needed(47) == 0 and second[0].first_needed(48) == 48 and not second[0].keeps_all
    assert second[1].shape == (2, 32, 16)
    arch, c = resolve_config(cases.folder_config(cases.CASE_B))
    needs = build_model(arch.plan(c)).cache_needs()
    assert [type(n) for n in leaf_needs(needs[1])] == [FixedState]  # one tap: no inputs are kept


# ------------------------------------------------------------------------------ the plain functions, read once more
def test_norms_and_activations_element_by_element():
    x, w = [0.5, -2.0, 3.0, 0.25], [0.1, -0.2, 0.0, 1.5]
    ms = sum(v * v for v in x) / 4
    got = plain.norm_one_plus(torch.tensor(x, dtype=F64), torch.tensor(w, dtype=F64), 1e-5)
    plain_got = plain.norm_plain(torch.tensor(x, dtype=F64), torch.tensor(w, dtype=F64), 1e-5)
    for i in range(4):
        assert abs(float(got[i]) - x[i] / math.sqrt(ms + 1e-5) * (1.0 + w[i])) < 1e-12
        assert abs(float(plain_got[i]) - x[i] / math.sqrt(ms + 1e-5) * w[i]) < 1e-12
    for z in (-3.0, -0.1, 0.0, 0.7, 4.0):
        want = 0.5 * z * (1.0 + math.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))
        assert abs(float(plain.gelu_tanh(torch.tensor(z, dtype=F64))) - want) < 1e-12
        assert abs(float(plain.silu(torch.tensor(z, dtype=F64))) - z / (1.0 + math.exp(-z))) < 1e-12


def test_convolution_by_hand_and_its_history():
    taps = torch.tensor([[0.5, -1.0, 2.0], [1.0, 0.0, -0.5]], dtype=F64)  # the last column is the current token's
    bias = torch.tensor([0.1, -0.2], dtype=F64)
    p = torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0], [7.0, 8.0]], dtype=F64)
    u, hist = plain.causal_conv(p, taps, bias, torch.zeros(2, 2, dtype=F64))
    assert u[0].tolist() == pytest.approx([2.0 * 1.0 + 0.1, -0.5 * 2.0 - 0.2])
    assert u[1].tolist() == pytest.approx([-1.0 * 1.0 + 2.0 * 3.0 + 0.1, -0.5 * 4.0 - 0.2])
    assert u[3].tolist() == pytest.approx([0.5 * 3.0 - 5.0 + 14.0 + 0.1, 4.0 - 4.0 - 0.2])
    assert hist.tolist() == [[5.0, 6.0], [7.0, 8.0]]
    a, h = plain.causal_conv(p[:1], taps, bias, torch.zeros(2, 2, dtype=F64))
    b, h = plain.causal_conv(p[1:], taps, bias, h)
    assert torch.allclose(torch.cat([a, b]), u)


def test_recurrent_unit_by_hand():
    """Two channels in two blocks of one, one tap: every number of two steps written out."""
    t64 = lambda v: torch.tensor(v, dtype=F64)
    w = {"m.y": t64([[1.0, 0.0], [0.0, 1.0]]), "m.y.b": t64([0.5, -0.5]),
         "m.x": t64([[2.0, 0.0], [0.0, -1.0]]), "m.x.b": t64([0.0, 0.25]),
         "m.conv": t64([[1.5], [0.5]]), "m.conv.b": t64([0.1, 0.0]),
         "m.ra": t64([[[0.7]], [[-0.3]]]), "m.ra.b": t64([[0.2], [0.0]]),
         "m.ri": t64([[[1.1]], [[0.4]]]), "m.ri.b": t64([[0.0], [-0.6]]),
         "m.lam": t64([-1.0, 0.5]), "m.o": t64([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]])}
    y = torch.tensor([[0.3, -1.2], [1.0, 0.4]], dtype=F64)
    out, (hist, s) = plain.recurrent_unit(y, w, "m", {"width": 2, "blocks": 2, "conv": 1})
    sig = lambda z: 1.0 / (1.0 + math.exp(-z))
    gelu = lambda z: 0.5 * z * (1.0 + math.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))
    state = [0.0, 0.0]
    ra, rab, ri, rib = [0.7, -0.3], [0.2, 0.0], [1.1, 0.4], [0.0, -0.6]
    xw, xb, yw, yb, cw, cb, lam = [2.0, -1.0], [0.0, 0.25], [1.0, 1.0], [0.5, -0.5], [1.5, 0.5], [0.1, 0.0], [-1.0, 0.5]
    for t in range(2):
        gated = []
        for c in range(2):
            u = cw[c] * (xw[c] * float(y[t, c]) + xb[c]) + cb[c]
            r, i = sig(ra[c] * u + rab[c]), sig(ri[c] * u + rib[c])
            a = math.exp(-8.0 * r * math.log1p(math.exp(lam[c])))
            state[c] = a * state[c] + math.sqrt(1.0 - a * a) * i * u  # from zero for the first token as for any other
            gated.append(state[c] * gelu(yw[c] * float(y[t, c]) + yb[c]))
        assert out[t].tolist() == pytest.approx([gated[0], gated[1], gated[0] + gated[1]], abs=1e-12)
    assert s.tolist() == pytest.approx(state) and hist.shape == (0, 2)


def test_rotation_pairs_neighbours_and_passes_the_rest():
    x = torch.arange(1.0, 13.0, dtype=F64).reshape(1, 2, 6)
    got = plain.rotate_pairs(x, [3], {"dims": 4, "base": 100.0})
    for h in range(2):
        for i in range(2):
            ang = 3 * 100.0 ** (-2.0 * i / 4)
            u, v = float(x[0, h, 2 * i]), float(x[0, h, 2 * i + 1])
            assert float(got[0, h, 2 * i]) == pytest.approx(u * math.cos(ang) - v * math.sin(ang))
            assert float(got[0, h, 2 * i + 1]) == pytest.approx(v * math.cos(ang) + u * math.sin(ang))
        assert got[0, h, 4:].tolist() == x[0, h, 4:].tolist()
    assert plain.rotate_pairs(x, [3], None) is x


def _attention_weights(width, heads, kv_heads, dim, vdim, seed):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g, dtype=F64)
    return {"m.q": r(heads * dim, width), "m.q.b": r(heads * dim), "m.k": r(kv_heads * dim, width), "m.k.b": r(kv_heads * dim),
            "m.v": r(kv_heads * vdim, width), "m.v.b": r(kv_heads * vdim), "m.q.norm": 1.0 + 0.1 * r(dim),
            "m.k.norm": 1.0 + 0.1 * r(dim), "m.g": r(heads * vdim, width), "m.o": r(width, heads * vdim)}


def test_attention_by_hand():
    """One query written out: biases, the norm per head with its shared weight, no rotation, the keys of its chunk
    only, kv heads shared by neighbouring query heads, the sigmoid gate on the heads side by side."""
    W, H, G, d, dv = 5, 4, 2, 4, 3
    w = _attention_weights(W, H, G, d, dv, 1)
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": 0.7, "mask": {"size": 3}}
    y = torch.randn(8, W, generator=torch.Generator().manual_seed(2), dtype=F64)
    out, _ = plain.chunk_attention(y, w, "m", m, 1e-6)
    t = 7  # sees positions 6 and 7
    heads_out = []
    for h in range(H):
        g = h // 2
        def normed(row, name):
            ms = sum(float(v) ** 2 for v in row) / d
            return [float(v) / math.sqrt(ms + 1e-6) * float(w[name][i]) for i, v in enumerate(row)]
        q = normed((w["m.q"] @ y[t] + w["m.q.b"])[h * d:(h + 1) * d], "m.q.norm")
        scores, values = [], []
        for j in (6, 7):
            k = normed((w["m.k"] @ y[j] + w["m.k.b"])[g * d:(g + 1) * d], "m.k.norm")
            scores.append(0.7 * sum(a * b for a, b in zip(q, k)))
            values.append((w["m.v"] @ y[j] + w["m.v.b"])[g * dv:(g + 1) * dv])
        e = [math.exp(s - max(scores)) for s in scores]
        heads_out += [sum(e[n] / sum(e) * float(values[n][i]) for n in range(2)) for i in range(dv)]
    gate = w["m.g"] @ y[t]
    gated = torch.tensor([v / (1.0 + math.exp(-float(gate[i]))) for i, v in enumerate(heads_out)], dtype=F64)
    assert torch.allclose(out[t], w["m.o"] @ gated, atol=1e-10)


def test_gated_linear_attention_by_hand():
    W, H, d, dv, rank, tau = 4, 2, 3, 2, 2, 4.0
    g = torch.Generator().manual_seed(3)
    r = lambda *s: torch.randn(*s, generator=g, dtype=F64)
    w = {"m.q": r(H * d, W), "m.k": r(H * d, W), "m.v": r(H * dv, W), "m.g": r(H * dv, W), "m.o": r(W, H * dv),
         "m.norm": 1.0 + 0.1 * r(dv), "m.a1": r(rank, W), "m.a2": r(H * d, rank), "m.a2.b": r(H * d)}
    y = r(5, W)
    out, S = plain.gated_linear_attention(y, w, "m", {"heads": H, "dim": d, "vdim": dv, "tau": tau}, 1e-6)
    state = [[[0.0] * dv for _ in range(d)] for _ in range(H)]
    for t in range(5):
        q, k, v = w["m.q"] @ y[t], w["m.k"] @ y[t], w["m.v"] @ y[t]
        z = w["m.a2"] @ (w["m.a1"] @ y[t]) + w["m.a2.b"]
        row = []
        for h in range(H):
            o = [0.0] * dv
            for i in range(d):
                alpha = (1.0 / (1.0 + math.exp(-float(z[h * d + i])))) ** (1.0 / tau)
                for j in range(dv):
                    state[h][i][j] = alpha * state[h][i][j] + float(k[h * d + i]) * float(v[h * dv + j])
                    o[j] += state[h][i][j] * float(q[h * d + i]) / math.sqrt(d)  # the read-out sees the token's own write
            ms = sum(x * x for x in o) / dv
            row += [o[j] / math.sqrt(ms + 1e-6) * float(w["m.norm"][j]) for j in range(dv)]
        gate = w["m.g"] @ y[t]
        gated = torch.tensor([x * float(gate[i]) / (1.0 + math.exp(-float(gate[i]))) for i, x in enumerate(row)], dtype=F64)
        assert torch.allclose(out[t], w["m.o"] @ gated, atol=1e-10), t
    assert torch.allclose(S, torch.tensor(state, dtype=F64), atol=1e-12)


def test_router_by_hand():
    """Eight outputs in four groups of two, two groups stay: the correction steers the choice and is no part of the
    weights; a group that is left out loses even its best output; identity experts are the last outputs."""
    w = {"m.router": torch.eye(8, dtype=F64), "m.correction": torch.tensor([0.0, 0.0, 0.5, 0.0, 0.0, 0.0, -0.9, 0.0], dtype=F64)}
    router = {"experts": 6, "identity": 2, "top": 3, "groups": {"count": 4, "keep": 2}}
    z = torch.tensor([2.0, 0.0, 0.1, -0.5, 1.0, 0.9, 3.0, 1.5], dtype=F64)
    s = [math.exp(float(v)) for v in z]
    s = [v / sum(s) for v in s]
    c = [s[i] + float(w["m.correction"][i]) for i in range(8)]
    # group scores: max(c0, c1), max(c2, c3), max(c4, c5), max(c6, c7): output 6 has the largest s and a choice score
    # below zero, so its group stands on output 7
    groups = sorted(range(4), key=lambda g: -max(c[2 * g], c[2 * g + 1]))[:2]
    allowed = sorted((i for i in range(8) if i // 2 in groups), key=lambda i: -c[i])[:3]
    chosen, weights, margin = plain.route(z, w, "m", router)
    assert chosen == allowed and set(groups) == {1, 0}
    total = sum(s[i] for i in allowed)
    assert [float(x) for x in weights] == pytest.approx([s[i] / total for i in allowed])
    assert margin > 0
    # every group stays: output 7 (an identity expert) is chosen, and its share of the result is the input itself
    chosen, weights, _ = plain.route(z, w, "m", dict(router, groups={"count": 4, "keep": 4}))
    assert chosen == [2, 0, 7]


def test_expert_and_mixture_by_hand():
    W, ff, L = 3, 2, 0.8
    g = torch.Generator().manual_seed(5)
    r = lambda *s: 2.0 * torch.randn(*s, generator=g, dtype=F64)
    w = {"m.e0.gate": r(ff, W), "m.e0.up": r(ff, W), "m.e0.down": r(W, ff), "m.router": r(3, W),
         "m.correction": torch.zeros(3, dtype=F64)}
    y = r(4, W)
    for t in range(4):
        a, b = w["m.e0.gate"] @ y[t], w["m.e0.up"] @ y[t]
        inner = []
        for j in range(ff):
            aj, bj = min(float(a[j]), L), max(-L, min(L, float(b[j])))  # the gate is capped from above only
            inner.append(aj / (1.0 + math.exp(-1.702 * aj)) * (bj + 1.0))
        assert torch.allclose(plain.expert(y[t], w, "m.e0", L), w["m.e0.down"] @ torch.tensor(inner, dtype=F64), atol=1e-12)
    mlp = {"kind": "moe", "expert": {"ff": ff, "limit": L}, "router": {"experts": 1, "identity": 2, "top": 2}}
    out = plain.mixture(y, w, "m", mlp)
    for t in range(4):
        chosen, weights, _ = plain.route(y[t], w, "m", mlp["router"])
        want = sum(float(g_) * (y[t] if e >= 1 else plain.expert(y[t], w, "m.e0", L)) for e, g_ in zip(chosen, weights))
        assert torch.allclose(out[t], want, atol=1e-12)
        assert sum(float(g_) for g_ in weights) == pytest.approx(1.0)


@pytest.mark.parametrize("case", sorted(cases.CASES))
def test_the_plain_implementation_cut_anywhere(case):
    cfg, weights = cases.folder_config(cases.CASES[case]), cases.make_weights(cases.CASES[case], 3)
    ids = cases.random_ids(cfg["vocab"], 60, 4)
    whole, _ = plain.forward(cfg, weights, ids)
    rng = random.Random(case)
    rows, state, pos = [], None, 0
    while pos < len(ids):
        n = min(len(ids) - pos, rng.choice([1, 1, 2, 5, 17]))
        part, state = plain.forward(cfg, weights, ids[pos:pos + n], start=pos, state=state)
        rows.append(part)
        pos += n
    assert torch.allclose(torch.cat(rows), whole, atol=1e-9, rtol=1e-9)


def test_a_safe_sequence_has_no_close_call():
    cfg, weights = cases.CASE_A, cases.make_weights(cases.CASE_A, 9)
    ids, rows = cases.safe_sequence(cfg, weights, 30, 1)
    margins = []
    logits, _ = plain.forward(cases.folder_config(cfg), weights, ids, margins=margins)
    assert min(margins) >= cases.CLOSE_CALL and torch.allclose(logits, rows, atol=1e-9)
