"""Samulorn without a GPU: the configuration reader and its refusals, the spec it emits (run order of
a loop, tensor names against the weights the tests make), and the plain implementation against
itself and against closed forms -- each mechanism alone, a prompt whole against the same prompt in
pieces down to one token."""
import copy
import math

import pytest
import torch
import torch.nn.functional as F

from plain_samulorn import (PlainSamulorn, causal_attention, delta_rule, dyt, gelu_tanh, over_rms,
                            rotary_frequencies, rotate_neighbours, route, short_conv)
from samulorn_helpers import (CONFIGS, SAMU_A, SAMU_B, SAMU_C, needle_model, needle_tokens, plain_logits,
                              random_tokens, weights_of)
from yalm_b200.config import ConfigError, config_from_dict
from yalm_b200.engine.lm import tensor_needs_of


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_spec_names_the_tests_weights(name):
    cfg_d, _ = CONFIGS[name]
    w = weights_of(name)
    cfg = config_from_dict(cfg_d).with_tensor_shapes({k: tuple(v.shape) for k, v in w.items()})
    needs = tensor_needs_of(cfg)
    assert sorted(needs) == sorted(w)
    for k, need in needs.items():
        assert tuple(need.shape) == tuple(w[k].shape), k
    spec = cfg.to_spec()
    assert [e.layer for e in spec.run_order] == PlainSamulorn(cfg_d, w).runs
    assert spec.head.tensors["weight"] == spec.embedding.tensors["weight"] == "embed"


def test_run_order_of_a_loop():
    order = lambda d: [e.layer for e in config_from_dict(d).to_spec().run_order]
    assert order(SAMU_A) == [0, 1, 2, 1, 2]
    assert order(SAMU_B) == [0, 1]
    assert order(SAMU_C) == [0, 1, 0, 1]
    d = copy.deepcopy(SAMU_A)
    d["loop"] = None
    assert order(d) == [0, 1, 2]
    d["loop"] = {"start": 0, "stop": 1, "times": 3}
    assert order(d) == [0, 0, 0, 1, 2]


def test_random_weights_mode_round_trip():
    cfg = config_from_dict(SAMU_A)
    again = config_from_dict(cfg.to_dict())
    assert sorted(tensor_needs_of(again)) == sorted(tensor_needs_of(cfg))
    assert again.to_dict()["layers"][0]["mixer"]["decay_rank"] > 0


@pytest.mark.parametrize("change, text", [
    (lambda d: d["layers"][0].update(type="window"), "type"),
    (lambda d: d["layers"][0]["mixer"].update(heads=3), "kv_heads"),
    (lambda d: d["layers"][1]["mixer"]["right"].update(blocks=5), "blocks"),
    (lambda d: d["layers"][1]["mixer"]["left"]["rot"].update(dims=15), "dims"),
    (lambda d: d["layers"][1]["mlp"]["router"].update(top=5), "top"),
    (lambda d: d["layers"][1]["mlp"].update(kind="soft"), "kind"),
    (lambda d: d["loop"].update(stop=9), "loop"),
    (lambda d: d.pop("norm"), "norm"),
    (lambda d: d["layers"][0]["mixer"].update(conv=1), "conv"),
])
def test_refusals(change, text):
    d = copy.deepcopy(SAMU_A)
    change(d)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(d)


# ------------------------------------------------------------------ the plain mechanisms
def test_plain_norms_and_activation():
    x = torch.randn(5, 7, dtype=torch.float64)
    w, b = torch.randn(7, dtype=torch.float64), torch.randn(7, dtype=torch.float64)
    assert torch.allclose(dyt(x, 0.3, w, b), torch.tanh(0.3 * x) * w + b)
    assert torch.allclose(over_rms(x, 0.0).pow(2).mean(-1), torch.ones(5, dtype=torch.float64))
    assert torch.allclose(gelu_tanh(x), F.gelu(x, approximate="tanh"))


def test_plain_short_conv_is_a_causal_convolution_with_a_state():
    g = torch.Generator().manual_seed(1)
    u, w = torch.randn(9, 5, generator=g, dtype=torch.float64), torch.randn(5, 4, generator=g, dtype=torch.float64)
    zeros = torch.zeros(3, 5, dtype=torch.float64)
    y, st = short_conv(u, w, zeros)
    ref = F.conv1d(F.pad(u.T[None], (3, 0)), w[:, None, :], groups=5)[0].T
    assert torch.allclose(y, ref)
    assert torch.equal(st, u[-3:])
    # the same in pieces, down to pieces shorter than the state
    out, state = [], zeros
    for a, b in ((0, 1), (1, 3), (3, 4), (4, 9)):
        piece, state = short_conv(u[a:b], w, state)
        out.append(piece)
    assert torch.allclose(torch.cat(out), y) and torch.equal(state, st)


def test_plain_rotation_bands_and_pairs():
    sc = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
    f0, f = rotary_frequencies(16, 1e4, None), rotary_frequencies(16, 1e4, sc)
    for i in range(8):
        wave = 2 * math.pi / float(f0[i])
        if wave < 64 / 4:
            assert f[i] == f0[i]
        elif wave > 64 / 1:
            assert math.isclose(float(f[i]), float(f0[i]) / 8.0)
        else:
            assert float(f0[i]) / 8.0 < float(f[i]) < float(f0[i])
    assert f[0] == f0[0] and f0[1] / 8.0 < f[1] < f0[1] and math.isclose(float(f[-1]), float(f0[-1]) / 8.0)
    x = torch.randn(3, 2, 12, dtype=torch.float64)
    pos = torch.tensor([0, 5, 9])
    y = rotate_neighbours(x, pos, rotary_frequencies(8, 1e4, None))
    assert torch.equal(y[..., 8:], x[..., 8:]) and torch.equal(y[0], x[0])          # the rest and position 0 pass
    assert torch.allclose(y.pow(2).sum(-1), x.pow(2).sum(-1))                        # pairs keep their length
    a = 5 * 1e4 ** (-2 / 8)                                                          # pair 1 = features (2, 3)
    assert torch.allclose(y[1, :, 2], x[1, :, 2] * math.cos(a) - x[1, :, 3] * math.sin(a), atol=1e-6)


def test_plain_delta_rule_writes_before_it_reads_and_forgets_by_channel():
    # orthonormal keys, beta 1, no decay: the state stores v under k and the read-out sees it at once
    dk, dv = 4, 3
    k = torch.eye(dk, dtype=torch.float64)
    v = torch.randn(dk, dv, dtype=torch.float64)
    S = torch.zeros(dk, dv, dtype=torch.float64)
    o = delta_rule(k.clone(), k, v, torch.ones(dk, dtype=torch.float64), torch.ones(dk, dk, dtype=torch.float64), S)
    assert torch.allclose(o, v) and torch.allclose(S, v)
    # writing the same key again with beta 1 replaces the value; a decay on one key channel fades that row only
    decay = torch.ones(1, dk, dtype=torch.float64)
    decay[0, 2] = 0.5
    o = delta_rule(k[:1].clone(), k[:1], v[1:2], torch.ones(1, dtype=torch.float64), decay, S)
    assert torch.allclose(S[0], v[1]) and torch.allclose(S[2], 0.5 * v[2]) and torch.allclose(S[3], v[3])


def test_plain_routing_rule():
    corr = torch.tensor([0.0, 0.0, -2.0, -2.0, 0.3, -1.0], dtype=torch.float64)
    z = torch.tensor([2.0, -3.0, 1.0, 0.9, 0.2, 3.0], dtype=torch.float64)
    # groups of two by the sum of both choices: (s0+s1), (s2+s3-4), (s4+s5-0.7); the second group's are negative
    chosen, w, margin = route(z, corr, 3, 2, 2, 2.5)
    s = torch.sigmoid(z)
    assert sorted(chosen.tolist()) == [0, 4]             # expert 5 has the largest score, but its choice is s - 1
    assert torch.allclose(w.sum(), torch.tensor(2.5, dtype=torch.float64))
    assert torch.allclose(w, s[chosen] / s[chosen].sum() * 2.5)
    assert margin > 0
    # a group that is not kept stays out even where its (negative) choices would beat nothing else: with one
    # group kept and top = 2, both experts of that group are taken, never one of a dropped group
    chosen, _, _ = route(z, corr - 5.0, 3, 1, 2, 1.0)
    assert sorted(chosen.tolist()) == [0, 1]


def test_plain_attention_is_causal_and_grouped():
    g = torch.Generator().manual_seed(3)
    q, k = torch.randn(6, 4, 8, generator=g, dtype=torch.float64), torch.randn(6, 2, 8, generator=g, dtype=torch.float64)
    v = torch.randn(6, 2, 5, generator=g, dtype=torch.float64)
    none = lambda d: torch.zeros(0, 2, d, dtype=torch.float64)
    o, K, V = causal_attention(q, k, v, none(8), none(5), 0.3)
    assert torch.allclose(o[0, 3], v[0, 1])                                  # the first token sees itself alone
    k2 = k.clone()
    k2[4:] += 1.0                                                            # later keys do not reach earlier queries
    o2, _, _ = causal_attention(q, k2, v, none(8), none(5), 0.3)
    assert torch.allclose(o2[:4], o[:4]) and not torch.allclose(o2[4:], o[4:])
    a, _, _ = causal_attention(q[:4], k[:4], v[:4], none(8), none(5), 0.3)
    b, _, _ = causal_attention(q[4:], k[4:], v[4:], k[:4], v[:4], 0.3)
    assert torch.allclose(torch.cat([a, b]), o)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_plain_whole_against_pieces(name):
    cfg, seed = CONFIGS[name]
    w = weights_of(name)
    toks = random_tokens(29, cfg["vocab"], seed)
    whole, _ = plain_logits(cfg, w, toks)
    for pieces in ([1] * 29, [2, 3, 1, 7], [28], [5, 24]):
        got, _ = plain_logits(cfg, w, toks, pieces)
        assert (got - whole).abs().max() <= 1e-5 * whole.abs().max(), pieces


def test_plain_needle_decides_the_probe():
    cfg, w = needle_model()
    toks = needle_tokens(300, 4, [120, 299])
    ref, _ = plain_logits(cfg, w, toks)
    without = list(toks)
    without[4] = 9
    other, _ = plain_logits(cfg, w, without)
    for p in (120, 299):
        assert (ref[p] - other[p]).abs().max() > 0.3 * ref[p].abs().max()
    assert (ref[50] - other[50]).abs().max() < 0.05                         # a token that does not ask barely moves
