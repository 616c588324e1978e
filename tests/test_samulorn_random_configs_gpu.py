"""Randomly drawn Samulorn configurations through the engine against the plain implementation: any
order of the two mixers, delta-rule layers with 1 to 6 heads over fewer q/k heads and key and value
sizes that are no multiple of 4, attention with key and value sizes from 8 to 128 that agree or
differ, rotation of nothing, a part of the head or all of it with and without band scaling,
convolutions of 2 to 5 taps, recurrent units in 1 to 5 blocks, experts in 1 to 4 groups with top
from 1 to all eligible ones, layers without feed-forward, a token input or none, loops over any run
of layers, widths and sizes that are no multiple of 8; prompts whole or cut in two, then tokens one
by one."""
import random

import pytest
import torch

from samulorn_helpers import (CLOSE_CALL, TOL, delta_layer, dense, make_weights, moe, parallel_layer, plain_logits,
                              random_tokens)

pytestmark = pytest.mark.gpu


def draw(seed):
    rng = random.Random(seed)
    layers, ranks = [], {}
    for i in range(rng.choice([1, 2, 3, 4])):
        r = rng.random()
        if r < 0.25:
            mlp = None
        elif r < 0.6:
            mlp = dense(rng.choice([8, 20, 48, 72, 130]))
        else:
            count = rng.choice([1, 2, 3, 4])
            per = rng.choice([1, 2, 3])
            keep = rng.randint(1, count)
            mlp = moe(count * per, count, keep, rng.randint(1, keep * per), rng.choice([8, 24, 40, 70]),
                      rng.choice([0.5, 1.0, 2.0]))
        if rng.random() < 0.5:
            G = rng.choice([1, 2, 3])
            layers.append(delta_layer(G * rng.choice([1, 2]), G, rng.choice([4, 8, 20, 33, 64, 128]),
                                      rng.choice([10, 16, 48, 64, 130]), rng.choice([2, 3, 4, 5]), mlp))
            ranks[i] = (rng.choice([1, 3, 8, 16, 40]), rng.choice([2, 5, 8, 24]))
        else:
            G = rng.choice([1, 2, 3])
            dim = rng.choice([8, 16, 24, 32, 64, 72, 96, 128])
            rot = None
            if rng.random() < 0.8:
                rot = {"base": rng.choice([100.0, 1e4, 1e6]), "dims": rng.choice([2, dim // 2 // 2 * 2 or 2, dim])}
                if rng.random() < 0.5:
                    rot["scaling"] = {"factor": rng.choice([2.0, 8.0, 32.0]), "low": 1.0, "high": rng.choice([2.0, 4.0]),
                                      "original": rng.choice([16, 64, 1024])}
            blocks = rng.choice([1, 2, 3, 5])
            layers.append(parallel_layer(G * rng.choice([1, 2, 4, 5]), G, dim, rng.choice([dim, dim, 8, 16, 40, 128]),
                                         rng.choice([2, 3, 4]), rng.choice([0.05, 0.2, dim ** -0.5]), rot,
                                         blocks * rng.choice([4, 8, 13, 32]), blocks, rng.choice([2, 4, 5]),
                                         rng.choice([0.5, 1.0, 1.2]), rng.choice([0.3, 1.0]), mlp))
    n = len(layers)
    cfg = {"architecture": "Samulorn", "vocab": rng.choice([61, 256, 500]), "width": rng.choice([24, 64, 72, 100, 136]),
           "norm": {"eps": rng.choice([1e-5, 1e-6])}, "embedding": {"scale": rng.choice([1.0, 4.0, 9.5])}, "layers": layers}
    if rng.random() < 0.6:
        cfg["token_side"] = {"dim": rng.choice([2, 8, 12, 16])}
    if rng.random() < 0.6:
        a = rng.randint(0, n - 1)
        b = rng.randint(a + 1, n)
        # at most six layer runs: a deeper stack of these small layers (heads normed over a handful of values)
        # turns 16-bit rounding into errors of the logits' own size, which tests nothing
        times = max(t for t in (1, 2, 3) if n + (t - 1) * (b - a) <= 6 or t == 1)
        cfg["loop"] = {"start": a, "stop": b, "times": rng.choice([1, times])}
    lens = [rng.randint(1, 230) for _ in range(rng.choice([1, 2, 3]))]
    return cfg, ranks, lens, rng.random() < 0.5


def page_budget(lens):
    return sum((n + 6 + 63) // 64 * 64 for n in lens)


@pytest.mark.parametrize("seed", range(40, 100))
def test_a_random_configuration_matches_the_plain_model(seed):
    from yalm_b200 import LM
    from yalm_b200.config import config_from_dict
    cfg, ranks, lens, cut = draw(seed)
    w = make_weights(cfg, 100 + seed, ranks=ranks)
    toks = [random_tokens(n + 6, cfg["vocab"], 7 * seed + i) for i, n in enumerate(lens)]
    refs, calls = [], []
    for t in toks:
        ref, m = plain_logits(cfg, w, t)
        refs.append(ref)
        # the routing decisions of a whole prompt come run by run, token by token within a run: the first
        # token with a close one bounds the positions a 16-bit run is held to
        close = [k % len(t) for k, v in enumerate(m.margins) if v < CLOSE_CALL]
        calls.append(min(close) if close else len(t))
    for dtype in ("float32", "bfloat16"):
        lm = LM(config_from_dict(cfg), dict(w), dtype=dtype, max_batch=len(lens), max_context=256,
                max_tokens=page_budget(lens))
        s = lm.acquire(len(lens))
        errs = []

        def see(logits, i, pos):
            assert bool(torch.isfinite(logits).all()), (dtype, cfg, lens, i, pos)
            if dtype != "float32" and pos >= calls[i]:
                return                                # after a routing call that 16 bits may decide the other way
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
        if not errs:
            continue
        worst = max(errs)
        if dtype == "float32":
            # a routing call within rounding of a tie may fall either way in 32 bits too: rows after one are left out
            margin_ok = all(c == len(t) for c, t in zip(calls, toks))
            bound = 10 * TOL[dtype]
            assert worst[0] <= bound or not margin_ok, (dtype, cfg, lens, cut, worst)
        else:
            # a drawn model may have a position whose head output nearly cancels, which a scale-free norm then
            # blows up from a rounding error to full size (a sequence's first delta-rule output is (k.q) u over
            # its own root mean square: the sign of a small k.q decides it): all but a few rows must be close
            if len(errs) < 4:
                continue
            errs.sort()
            assert errs[len(errs) * 3 // 4][0] <= TOL[dtype], (dtype, cfg, lens, cut, errs[-3:])
