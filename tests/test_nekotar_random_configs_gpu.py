"""Randomly drawn Nekotar configurations through the engine against the plain implementation:
any order of the three mixers, 1 to 5 residual copies, wkv layers with 1 to 5 heads and key
sizes that are no multiple of 4, latent layers whose sizes agree or differ (and layers that read
an earlier layer's latent with heads and sizes of their own), windowed layers with key and
value sizes from 8 to 128, rotation of a part of the head or all of it, windows from 1 position
to longer than the prompts, no kept position up to more than the prompt has, widths and
feed-forward sizes that are no multiple of 8, layers without feed-forward; prompts whole or cut
in two, then tokens one by one."""
import random

import pytest
import torch

from nekotar_helpers import TOL, latent_layer, make_weights, random_tokens, window_layer, wkv_layer
from plain_nekotar import plain_forward

pytestmark = pytest.mark.gpu


def draw(seed):
    rng = random.Random(seed)
    layers, ranks, owners = [], {}, []
    for i in range(rng.choice([1, 2, 3, 4, 5])):
        ff = None if rng.random() < 0.3 else rng.choice([8, 20, 48, 72, 130])
        kind = rng.choice(["wkv", "latent", "latent", "window"])
        if kind == "wkv":
            layers.append(wkv_layer(rng.choice([1, 2, 3, 5]), rng.choice([4, 8, 20, 33, 64, 128]), ff))
            ranks[i] = rng.choice([1, 3, 8, 16, 40])
        elif kind == "latent":
            H, dim, vdim = rng.choice([1, 2, 3, 6]), rng.choice([8, 16, 24, 40, 64]), rng.choice([8, 12, 32, 64])
            scale = rng.choice([0.05, 0.2, dim ** -0.5])
            if owners and rng.random() < 0.5:
                src = rng.choice(owners)
                m = layers[src]["mixer"]
                layers.append(latent_layer(H, dim, m["rot_dim"], vdim, m["kv_rank"], scale, m["rot"]["base"], ff, kv_from=src))
            else:
                owners.append(i)
                layers.append(latent_layer(H, dim, rng.choice([2, 8, 16, 32, 64]), vdim,
                                           rng.choice([8, 20, 48, 96, 128, 190]), scale, rng.choice([100.0, 1e4, 2e4]), ff))
        else:
            G = rng.choice([1, 2, 3])
            dim = rng.choice([8, 16, 24, 32, 64, 72, 96, 128])
            layers.append(window_layer(G * rng.choice([1, 2, 4, 5]), G, dim, rng.choice([dim, dim, 8, 16, 32, 40, 128]),
                                       rng.choice([0.05, 0.2, dim ** -0.5]), rng.choice([1, 2, 7, 33, 40, 64, 65, 100, 400]),
                                       rng.choice([0, 1, 3, 20, 64, 70, 300]), rng.choice([100.0, 1e4, 1e6]),
                                       rng.choice([2, dim // 2 // 2 * 2 or 2, dim]), ff))
    cfg = {"architecture": "Nekotar", "vocab": rng.choice([61, 256, 500]), "width": rng.choice([24, 64, 72, 100, 136]),
           "norm": {"eps": rng.choice([1e-5, 1e-6])}, "residual_mult": rng.choice([0.25, 0.5, 1.0, 1.5]),
           "streams": rng.choice([1, 2, 3, 4, 5]), "layers": layers}
    lens = [rng.randint(1, 230) for _ in range(rng.choice([1, 2, 3]))]
    return cfg, ranks, lens, rng.random() < 0.5


def page_budget(lens):
    return sum((n + 6 + 63) // 64 * 64 for n in lens)


@pytest.mark.parametrize("seed", range(60, 90))
def test_a_random_configuration_matches_the_plain_model(seed):
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    cfg, ranks, lens, cut = draw(seed)
    w = make_weights(cfg, 100 + seed, decay_ranks=ranks)
    toks = [random_tokens(n + 6, cfg["vocab"], 7 * seed + i) for i, n in enumerate(lens)]
    refs = [plain_forward(cfg, w, t) for t in toks]
    for dtype in ("float32", "bfloat16"):
        lm = LM(config_from_dict(cfg), dict(w), dtype=dtype, max_batch=len(lens), max_context=256,
                max_tokens=page_budget(lens))
        s = lm.acquire(len(lens))
        errs = []

        def see(logits, i, pos):
            assert bool(torch.isfinite(logits).all()), (dtype, cfg, lens, i, pos)
            errs.append((float((logits - refs[i][pos]).abs().max() / refs[i].abs().max()), i, pos))

        if cut:
            first = [max(1, n // 2) for n in lens]
            lg = lm.step([t[:c] for t, c in zip(toks, first)], s, [[c - 1] for c in first]).cpu()
            for i, c in enumerate(first):
                see(lg[i], i, c - 1)
            rest = [i for i, (c, n) in enumerate(zip(first, lens)) if n > c]
            if rest:
                lg = lm.step([toks[i][first[i]:lens[i]] for i in rest], [s[i] for i in rest],
                             [[lens[i] - first[i] - 1] for i in rest]).cpu()
                for k, i in enumerate(rest):
                    see(lg[k], i, lens[i] - 1)
        else:
            lg = lm.step([t[:n] for t, n in zip(toks, lens)], s, [[0, n - 1] for n in lens]).cpu()
            for i, n in enumerate(lens):
                see(lg[2 * i], i, 0)
                see(lg[2 * i + 1], i, n - 1)
        for k in range(6):
            lg = lm.step([[t[n + k]] for t, n in zip(toks, lens)], s, [[0]] * len(lens)).cpu()
            for i, n in enumerate(lens):
                see(lg[i], i, n + k)
        lm.release(s)
        lm.rt.check_status()
        worst = max(errs)
        if dtype == "float32":
            assert worst[0] <= 10 * TOL[dtype], (dtype, cfg, lens, cut, worst)
        else:
            # a drawn model may have a position whose sublayer output nearly cancels, which the scale-free
            # norm of a wkv head then blows up from a rounding error to full size: all but a few rows must be close
            errs.sort()
            assert errs[len(errs) * 3 // 4][0] <= TOL[dtype], (dtype, cfg, lens, cut, errs[-3:])
