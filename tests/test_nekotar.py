"""Nekotar without a GPU: the configuration reader and its refusals, the tensors the model
declares, the plain implementation's own mechanisms (the kept-first window's edges, rotation
layouts, the wkv recurrence carried by hand, the latent attention in its absorbed form, residual
copies that reduce to the plain sum), and that the crafted one-key models do show a mask that is
one position off or a far key that is lost."""
import copy

import pytest
import torch

from nekotar_helpers import (CONFIGS, DECAY_RANKS, NEKO_A, NEKO_B, PROBE, make_weights, needle_model,
                             needle_tokens, random_tokens, weights_of, with_mask)
from plain_nekotar import (plain_forward, plain_kept_window_mask, plain_latent, plain_latent_attention,
                           plain_norm, plain_rotate, plain_sublayer, plain_wkv)
from yalm_b200.config import ConfigError, config_from_dict
from yalm_b200.config.nekotar import NekotarConfig
from yalm_b200.engine.lm import tensor_needs_of


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_declared_tensors_are_the_checkpoint_names(name):
    cfg, _ = CONFIGS[name]
    w = weights_of(name)
    c = config_from_dict(cfg)
    assert isinstance(c, NekotarConfig)
    c = c.with_tensor_shapes({k: tuple(v.shape) for k, v in w.items()})
    assert [c.layers[i].decay_rank for i in sorted(DECAY_RANKS[name])] == [DECAY_RANKS[name][i] for i in sorted(DECAY_RANKS[name])]
    needs = tensor_needs_of(c)
    assert {k: tuple(v.shape) for k, v in needs.items()} == {k: tuple(v.shape) for k, v in w.items()}
    # what the reader writes back reads as the same model
    again = config_from_dict(c.to_dict())
    assert again.to_spec().layers == c.to_spec().layers


def test_spec_carries_every_constant():
    spec = config_from_dict(NEKO_A).to_spec()
    assert [l.block for l in spec.layers] == ["hyper_prenorm"] * 5
    assert spec.embedding.params["norm"] == {"eps": 1e-5}
    first = spec.layers[0]
    n = first.part("mixer_norm")
    assert n.kind == "hyper_rmsnorm" and n.params["copies"] == 3 and n.params["residual_scale"] == 0.7
    assert n.tensors == {"weight": "l0.norm1", "in": "l0.hc1.in", "out": "l0.hc1.out", "mix": "l0.hc1.mix"}
    assert first.part("mixer").kind == "wkv_time_mix" and first.part("mixer").params["key_dim"] == 16
    lat = spec.layers[1].part("mixer").params
    assert (lat["head_dim"], lat["rot_dim"], lat["value_dim"], lat["kv_rank"], lat["scale"], lat["rot_base"],
            lat["owns_latent"]) == (16, 8, 24, 40, 0.2, 1e4, True)
    assert "feed_forward" not in spec.layers[1].parts
    att = spec.layers[2].part("mixer").params
    assert (att["window"], att["keep_first"], att["head_dim"], att["value_dim"], att["bias"]) == (24, 5, 16, 32, True)
    assert att["position"].params["layout"] == "halves" and att["position"].params["dims"] == 8
    shared = spec.layers[3].part("mixer")
    assert not shared.params["owns_latent"] and "l3.mix.dkv" not in shared.tensors.values()
    assert [(e.layer, e.reads_cache_of) for e in spec.run_order] == [(0, None), (1, None), (2, None), (3, 1), (4, None)]
    c = config_from_dict(NEKO_A)
    assert c.ignorable_tensor("l1.norm2") and c.ignorable_tensor("l4.hc2.mix") and not c.ignorable_tensor("l0.norm2")


def test_refusals():
    def broken(change, cfg=NEKO_A):
        c = copy.deepcopy(cfg)
        change(c)
        with pytest.raises(ConfigError):
            config_from_dict(c)
    broken(lambda c: c["layers"][0].update(type="convolution"))
    broken(lambda c: c["layers"][2]["mixer"].update(kv_heads=3))             # 4 heads over 3
    broken(lambda c: c["layers"][2]["mixer"]["rot"].update(dims=18))          # more than the head has
    broken(lambda c: c["layers"][2]["mixer"]["mask"].update(size=0))
    broken(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=4))           # the rotated part is rot_dim
    broken(lambda c: c["layers"][3]["mixer"].update(kv_from=2))               # not a latent layer
    broken(lambda c: c["layers"][3]["mixer"].update(kv_from=3))               # itself
    broken(lambda c: c["layers"][3]["mixer"].update(kv_rank=48))              # another row than its source's
    broken(lambda c: c["layers"][0]["mlp"].update(kind="moe"))
    broken(lambda c: c.update(streams=0))
    broken(lambda c: c.pop("norm"))
    broken(lambda c: c.update(layers=[]))


def test_kept_window_edges():
    size, keep, T = 5, 3, 20
    m = plain_kept_window_mask(T, size, keep)
    for i in range(T):
        for j in range(T):
            assert bool(m[i, j]) == (j <= i and (j > i - size or j < keep))
    assert m[9, 5] and not m[9, 4] and not m[9, 3] and m[9, 2] and m[19, 0]
    # more kept positions than the window is long: no gap until the kept ones end
    m = plain_kept_window_mask(30, 4, 10)
    assert m[12, 9] and m[13, 9] and not m[14, 10] and m[14, 11]
    assert torch.equal(plain_kept_window_mask(12, 4, 0), torch.tril(torch.ones(12, 12)).bool() & ~torch.tril(torch.ones(12, 12), -4).bool())


def test_rotation_layouts():
    u = torch.randn(6, 2, 12, dtype=torch.float64)
    pos = torch.arange(6)
    a, b = plain_rotate(u, pos, 100.0, 8, neighbours=True), plain_rotate(u, pos, 100.0, 8, neighbours=False)
    assert torch.equal(a[..., 8:], u[..., 8:]) and torch.equal(b[..., 8:], u[..., 8:])
    assert torch.allclose(a[0], u[0]) and torch.allclose(b[0], u[0])            # position 0 turns nothing
    # both layouts turn the same pairs by the same angles, only stored in another order
    v = u.clone()
    v[..., :8] = u[..., [0, 4, 1, 5, 2, 6, 3, 7]]
    assert torch.allclose(plain_rotate(v, pos, 100.0, 8, neighbours=True)[..., [0, 2, 4, 6, 1, 3, 5, 7]], b[..., :8], atol=1e-6)
    # a rotation keeps lengths, and positions offset by the same amount keep q.k
    assert torch.allclose(a.norm(dim=-1), u.norm(dim=-1))
    q, k = torch.randn(1, 1, 8, dtype=torch.float64), torch.randn(1, 1, 8, dtype=torch.float64)
    dot = lambda i, j: float((plain_rotate(q, torch.tensor([i]), 50.0, 8, True) * plain_rotate(k, torch.tensor([j]), 50.0, 8, True)).sum())
    assert abs(dot(7, 3) - dot(104, 100)) < 1e-5


def test_wkv_recurrence_by_hand():
    cfg, seed = CONFIGS["neko_a"]
    w = {k: v.double() for k, v in weights_of("neko_a").items()}
    m, p, D = cfg["layers"][0]["mixer"], "l0.mix", cfg["width"]
    H, d = m["heads"], m["dim"]
    h = torch.randn(11, D, dtype=torch.float64)
    whole = plain_wkv(w, p, m, h, 1e-5)
    # the same token by token with the state and the previous input handed on, the bonus as a dot product
    S, prev, rows = torch.zeros(H, d, d, dtype=torch.float64), torch.zeros(D, dtype=torch.float64), []
    for t in range(11):
        x = h[t]
        mix = {s: x + (prev - x) * w[f"{p}.mu.{s}"] for s in "rkvgw"}
        r, k, v = [(w[f"{p}.{s}"] @ mix[s]).view(H, d) for s in "rkv"]
        gate = torch.nn.functional.silu(w[f"{p}.g"] @ mix["g"])
        decay = torch.exp(-torch.exp(w[f"{p}.w2"] @ torch.tanh(w[f"{p}.w1"] @ mix["w"]) + w[f"{p}.w0"])).view(H, d)
        o = torch.einsum("hkv,hk->hv", S, r) + (r * w[f"{p}.u"] * k).sum(-1, keepdim=True) * v
        S = decay[:, :, None] * S + k[:, :, None] * v[:, None, :]
        o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + 1e-5)
        rows.append(w[f"{p}.o"] @ (o.reshape(-1) * w[f"{p}.norm"] * gate))
        prev = x
    assert torch.allclose(whole, torch.stack(rows), atol=1e-10)
    # a sequence that starts later starts from nothing: the first token sees no previous input and no state
    assert torch.allclose(plain_wkv(w, p, m, h[:1], 1e-5), whole[:1], atol=1e-12)
    assert not torch.allclose(plain_wkv(w, p, m, h[5:6], 1e-5), whole[5:6], atol=1e-3)


def test_latent_attention_in_its_absorbed_form():
    """Keys and values of all heads are functions of one row [c | kr]: moving the queries into the
    latent space and expanding the mixed latent afterwards gives the same output."""
    cfg, _ = CONFIGS["neko_a"]
    w = {k: v.double() for k, v in weights_of("neko_a").items()}
    m, p = cfg["layers"][1]["mixer"], "l1.mix"
    H, d, rd, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = 9
    h = torch.randn(T, cfg["width"], dtype=torch.float64)
    c, kr = plain_latent(w, p, m, h, 1e-5)
    ref = plain_latent_attention(w, p, m, h, c, kr)
    q = (h @ w[f"{p}.q"].T).view(T, H, d + rd)
    q_rot = plain_rotate(q[..., d:], torch.arange(T), m["rot"]["base"], rd, neighbours=True)
    q_lat = torch.einsum("thd,hdr->thr", q[..., :d], w[f"{p}.uk"].view(H, d, R))
    s = (torch.einsum("ihr,jr->hij", q_lat, c) + torch.einsum("ihd,jd->hij", q_rot, kr)) * m["scale"]
    s = s.masked_fill(~torch.tril(torch.ones(T, T)).bool()[None], float("-inf"))
    mixed = torch.einsum("hij,jr->ihr", torch.softmax(s, -1), c)
    o = torch.einsum("ihr,hvr->ihv", mixed, w[f"{p}.uv"].view(H, dv, R)).reshape(T, H * dv)
    got = (o * torch.sigmoid(h @ w[f"{p}.g"].T)) @ w[f"{p}.o"].T
    assert torch.allclose(got, ref, atol=1e-10)
    # the latent is normed, the rotated key part is not
    z = h @ w[f"{p}.dkv"].T
    assert torch.allclose(c, plain_norm(z[:, :R], w[f"{p}.dkv.norm"], 1e-5))
    assert torch.allclose(kr[0], z[0, R:])                                    # position 0 turns nothing


def test_one_residual_copy_is_the_plain_sum():
    D, T = 16, 5
    X = torch.randn(1, T, D, dtype=torch.float64)
    wn = torch.rand(D, dtype=torch.float64) + 0.5
    w = {"hc.in": torch.ones(1), "hc.out": torch.ones(1), "hc.mix": torch.ones(1, 1)}
    f = lambda h: 2.0 * h + 1.0
    new = plain_sublayer(w, "hc", X, wn, 1e-6, 0.5, f)
    assert torch.allclose(new[0], X[0] + 0.5 * f(plain_norm(X[0], wn, 1e-6)))
    # several copies: every new copy is formed from the OLD ones
    s = 3
    X = torch.randn(s, T, D, dtype=torch.float64)
    w = {"hc.in": torch.randn(s), "hc.out": torch.randn(s), "hc.mix": torch.randn(s, s)}
    new = plain_sublayer(w, "hc", X, wn, 1e-6, 0.7, f)
    y = f(plain_norm(sum(w["hc.in"][i].double() * X[i] for i in range(s)), wn, 1e-6))
    for j in range(s):
        want = sum(w["hc.mix"][i, j].double() * X[i] for i in range(s)) + 0.7 * w["hc.out"][j].double() * y
        assert torch.allclose(new[j], want)


@pytest.mark.parametrize("size, keep", [(9, 4), (9, 12)])
def test_the_crafted_window_model_shows_a_mask_that_is_one_off(size, keep):
    cfg, w = needle_model("attention", size, keep)
    n = 60
    for at, sees_for_ever in ((keep - 1, True), (keep, False)):
        edge = at + size                                    # the first position that the window no longer covers
        toks = needle_tokens(n, at, [edge - 1, edge, n - 2])
        ref = plain_forward(cfg, w, toks)
        scale = float(ref.abs().max())
        differs = lambda other, pos: float((other[pos] - ref[pos]).abs().max()) / scale > 0.05
        longer = plain_forward(with_mask(cfg, size=size + 1), w, toks)
        shorter = plain_forward(with_mask(cfg, size=size - 1), w, toks)
        if sees_for_ever:                                   # the last kept position: the window's length does not matter
            assert not differs(longer, edge) and not differs(shorter, edge - 1)
            assert differs(plain_forward(with_mask(cfg, keep_first=keep - 1), w, toks), n - 2)
        else:                                               # the first position that is not kept
            assert differs(longer, edge) and differs(shorter, edge - 1)
            assert differs(plain_forward(with_mask(cfg, keep_first=keep + 1), w, toks), n - 2)
        assert not differs(longer, edge - 1)


@pytest.mark.parametrize("kind", ["latent", "shared_latent"])
def test_the_crafted_latent_model_shows_a_lost_far_key(kind):
    cfg, w = needle_model(kind)
    n = 300
    toks = needle_tokens(n, 3, [n - 2])
    ref = plain_forward(cfg, w, toks)
    gone = list(toks)
    gone[3] = 9                                             # an ordinary token in the needle's place
    other = plain_forward(cfg, w, gone)
    assert float((other[n - 2] - ref[n - 2]).abs().max()) / float(ref.abs().max()) > 0.05
    assert float((other[n - 3] - ref[n - 3]).abs().max()) / float(ref.abs().max()) < 0.02


def test_other_sizes_run_through_the_plain_model():
    for name, (cfg, seed) in CONFIGS.items():
        w = weights_of(name)
        toks = random_tokens(40, cfg["vocab"], seed)
        outs = []
        lg = plain_forward(cfg, w, toks, layer_outputs=outs)
        assert lg.shape == (40, cfg["vocab"]) and bool(torch.isfinite(lg).all()) and len(outs) == len(cfg["layers"])
        # causal: a prefix's logits do not depend on what follows
        assert torch.allclose(plain_forward(cfg, w, toks[:17]), lg[:17], atol=1e-9)
