"""Shared pieces of the Samulorn tests: small configurations that differ from each other in every
size and option (also values that a model may happen to make equal or 1), random weights by
checkpoint name, references from the plain implementation in 64 bits, and a crafted model in which
ONE far key decides a logit."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from plain_samulorn import PlainSamulorn


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, count, keep, top, ff, scale):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "groups": {"count": count, "keep": keep}, "top": top, "scale": scale}}


def delta_layer(heads, kv, dim, vdim, conv, mlp):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": mlp}


def parallel_layer(heads, kv, dim, vdim, conv, scale, rot, width, blocks, rconv, ls, rs, mlp):
    left = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv, "scale": scale}
    if rot is not None:
        left["rot"] = rot
    return {"type": "parallel", "mixer": {"left": left, "right": {"width": width, "blocks": blocks, "conv": rconv},
                                          "left_scale": ls, "right_scale": rs}, "mlp": mlp}


# a loop over two layers, fewer q/k heads than value heads in the delta rule, value heads narrower and
# wider than key heads, half a head rotated with band scaling, experts in groups, a layer without mlp
SAMU_A = {
    "architecture": "Samulorn", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 6.0},
    "token_side": {"dim": 8}, "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [delta_layer(4, 2, 16, 24, 3, dense(96)),
               parallel_layer(4, 2, 32, 16, 2, 0.2, {"base": 1e4, "dims": 16, "scaling": {
                   "factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}}, 48, 3, 4, 0.8, 1.3,
                   moe(6, 3, 2, 2, 40, 1.5)),
               delta_layer(2, 2, 32, 32, 4, None)],
}
# no loop, no token input, everything that can be 1: one kv head, one group, top 1, one block; head
# size 64 rotated in full without scaling (the tensor-core prompt attention); loop times 1
SAMU_B = {
    "architecture": "Samulorn", "vocab": 300, "width": 96, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
    "loop": {"start": 0, "stop": 1, "times": 1},
    "layers": [parallel_layer(3, 1, 64, 64, 4, 0.125, {"base": 5e5, "dims": 64}, 64, 1, 2, 1.0, 1.0,
                              moe(3, 1, 1, 1, 48, 1.0)),
               delta_layer(1, 1, 64, 48, 2, dense(128))],
}
# a width that is no multiple of 8 (products on the FMA kernel), sizes that are no multiple of 4, no
# rotation at all, low-rank sizes 5 and 6, top = all experts of the kept group, a loop over every layer
SAMU_C = {
    "architecture": "Samulorn", "vocab": 130, "width": 100, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
    "token_side": {"dim": 6}, "loop": {"start": 0, "stop": 2, "times": 2},
    "layers": [delta_layer(3, 1, 20, 10, 4, moe(4, 2, 1, 2, 30, 1.25)),
               parallel_layer(2, 2, 24, 40, 3, 0.3, None, 30, 5, 3, 1.2, 0.5, dense(50))],
}
RANKS = {"samu_a": {0: (8, 16), 2: (4, 4)}, "samu_b": {1: (16, 8)}, "samu_c": {0: (5, 6)}}
CONFIGS = {"samu_a": (SAMU_A, 11), "samu_b": (SAMU_B, 22), "samu_c": (SAMU_C, 33)}

# Largest logit error relative to the request's largest logit.
TOL = {"float32": 1e-4, "bfloat16": 6e-2, "float16": 8e-3}
# The third configuration divides heads of 10 values by their own root mean square and repeats its
# layers: where such a head nearly cancels, a 16-bit rounding error comes out at full size (its median
# error is a seventh of the bound above; single rows reach it).
TOL_OF = {"samu_c": {"float32": 1e-4, "bfloat16": 1e-1, "float16": 1.3e-2}}
# a routing decision closer than this (in score units) may fall the other way in 16 bits
CLOSE_CALL = 0.05


def make_weights(cfg: dict, seed: int, dtype=torch.bfloat16, ranks: Optional[Dict[int, tuple]] = None
                 ) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    D, V = cfg["width"], cfg["vocab"]
    mat = lambda r, c, std: (std * torch.randn(r, c, generator=g)).to(dtype)
    vec = lambda n, std: (std * torch.randn(n, generator=g)).to(dtype)
    ones = lambda n: (1.0 + 0.1 * torch.randn(n, generator=g)).to(dtype)
    a = D ** -0.5
    w = {"embed": mat(V, D, 0.3)}

    def tanh_norm(name, alpha):
        w[name], w[name + ".b"] = ones(D), vec(D, 0.05)
        w[name + ".alpha"] = torch.tensor(alpha + 0.1 * torch.rand((), generator=g).item()).to(dtype)

    def conv(name, rows, taps):
        w[name] = (0.4 * torch.randn(rows, taps, generator=g) + torch.eye(taps)[-1]).to(dtype)

    tanh_norm("final.norm", 0.4)
    side = (cfg.get("token_side") or {}).get("dim", 0)
    if side:
        w["side.embed"] = mat(V, side * len(cfg["layers"]), 1.0)
    for i, layer in enumerate(cfg["layers"]):
        p, m, q = f"l{i}", layer["mixer"], f"l{i}.mix"
        tanh_norm(f"{p}.norm1", 0.5)
        tanh_norm(f"{p}.norm1b", 0.7)
        if layer["type"] == "channel_delta":
            H, G, dk, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            ra, rg = (ranks or {}).get(i, (8, 8))
            for name, rows in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                w[f"{q}.{name}"] = mat(rows, D, 3.0 * a)
                conv(f"{q}.{name}.conv", rows, taps)
            w[f"{q}.b"] = mat(H, D, 2.0 * a)
            # decays from nearly 1 (a state that remembers hundreds of tokens) down to a few tokens
            w[f"{q}.A_log"] = (-5.0 + 5.0 * torch.rand(H, generator=g)).to(dtype)
            w[f"{q}.a1"], w[f"{q}.a2"] = mat(ra, D, 2.0 * a), mat(H * dk, ra, ra ** -0.5)
            w[f"{q}.dt_bias"] = vec(H * dk, 1.0)
            w[f"{q}.g1"], w[f"{q}.g2"] = mat(rg, D, 2.0 * a), mat(H * dv, rg, rg ** -0.5)
            w[f"{q}.norm"] = ones(dv)
            w[f"{q}.o"] = mat(D, H * dv, 2.0 * (H * dv) ** -0.5)
        else:
            left, right = m["left"], m["right"]
            H, G, d, dv, taps = left["heads"], left["kv_heads"], left["dim"], left["vdim"], left["conv"]
            for name, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                w[f"{q}.left.{name}"] = mat(rows, D, 3.0 * a)
                w[f"{q}.left.{name}.b"] = vec(rows, 0.3)
                conv(f"{q}.left.{name}.conv", rows, taps)
            w[f"{q}.left.o"] = mat(D, H * dv, 2.0 * (H * dv) ** -0.5)
            W, B = right["width"], right["blocks"]
            bw = W // B
            for name in ("y", "x"):
                w[f"{q}.right.{name}"] = mat(W, D, 3.0 * a)
                w[f"{q}.right.{name}.b"] = vec(W, 0.3)
            conv(f"{q}.right.conv", W, right["conv"])
            w[f"{q}.right.conv.b"] = vec(W, 0.2)
            for name in ("ra", "ri"):
                w[f"{q}.right.{name}"] = (bw ** -0.5 * torch.randn(B, bw, bw, generator=g)).to(dtype)
                w[f"{q}.right.{name}.b"] = (0.5 * torch.randn(B, bw, generator=g)).to(dtype)
            # softplus(lam) from 0.002 (a state that lives for hundreds of tokens) to about 1
            w[f"{q}.right.lam"] = (-6.0 + 6.5 * torch.rand(W, generator=g)).to(dtype)
            w[f"{q}.right.o"] = mat(D, W, 2.0 * W ** -0.5)
        mlp = layer["mlp"]
        if mlp:
            tanh_norm(f"{p}.norm2", 0.5)
            tanh_norm(f"{p}.norm2b", 0.7)
            if mlp["kind"] == "dense":
                ff = mlp["ff"]
                w[f"{p}.mlp.gate"], w[f"{p}.mlp.up"] = mat(ff, D, 2.0 * a), mat(ff, D, 2.0 * a)
                w[f"{p}.mlp.down"] = mat(D, ff, 2.0 * ff ** -0.5)
            else:
                E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
                w[f"{p}.mlp.router"] = mat(E, D, 6.0 * a)
                # offsets large enough to turn choice scores negative and to move the choice
                w[f"{p}.mlp.correction"] = (-0.6 + 0.5 * torch.randn(E, generator=g)).to(dtype)
                for j in range(E):
                    w[f"{p}.mlp.e{j}.gate"], w[f"{p}.mlp.e{j}.up"] = mat(ff, D, 2.0 * a), mat(ff, D, 2.0 * a)
                    w[f"{p}.mlp.e{j}.down"] = mat(D, ff, 2.0 * ff ** -0.5)
        if side:
            w[f"{p}.side.gate"], w[f"{p}.side.proj"] = mat(side, D, 2.0 * a), mat(D, side, side ** -0.5)
            w[f"{p}.side.norm"] = (0.5 + 0.05 * torch.randn(D, generator=g)).to(dtype)
    return w


def weights_of(name: str, dtype=torch.bfloat16):
    cfg, seed = CONFIGS[name]
    return make_weights(cfg, seed, dtype, RANKS[name])


def random_tokens(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def plain_logits(cfg, w, toks, pieces=None, taps=None) -> torch.Tensor:
    """Logits [len(toks), vocab] of the plain implementation in 64 bits, the prompt fed whole or in
    the given pieces."""
    m = PlainSamulorn(cfg, w, torch.float64)
    m.taps = taps
    st = m.new_state()
    out, at = [], 0
    for n in (pieces or [len(toks)]):
        out.append(m.forward(toks[at:at + n], st))
        at += n
    if at < len(toks):
        out.append(m.forward(toks[at:], st))
    return torch.cat(out).float(), m


def safe_tokens(cfg, w, n: int, seed: int):
    """n random tokens, drawn one after the other so that no routing decision of the plain
    implementation is a close call (a token that brings one is drawn again), and their reference logits."""
    import copy
    g = torch.Generator().manual_seed(seed)
    m = PlainSamulorn(cfg, w, torch.float64)
    st = m.new_state()
    toks, rows = [], []
    while len(toks) < n:
        for _ in range(200):
            t = int(torch.randint(0, cfg["vocab"], (1,), generator=g))
            trial = copy.deepcopy(st)
            m.margins = []
            row = m.forward([t], trial)
            if not m.margins or min(m.margins) >= CLOSE_CALL:
                break
        else:
            raise AssertionError("no token without a close routing call was found")
        st = trial
        toks.append(t)
        rows.append(row[0])
    return toks, torch.stack(rows).float()


def plain_generate_greedy(cfg, w, prompt: List[int], n_new: int) -> List[int]:
    m = PlainSamulorn(cfg, w, torch.float64)
    st = m.new_state()
    logits = m.forward(list(prompt), st)
    out = []
    for _ in range(n_new):
        out.append(int(logits[-1].argmax()))
        logits = m.forward([out[-1]], st)
    return out


def add_portions(tr, rid: str, toks: List[int], sizes: List[int], tag="p"):
    """One request whose prompt comes in portions of the given sizes (the last takes the rest),
    logits at every position."""
    name, at = f"{tag}-{rid}", 0
    tr.need([len(toks)])
    cuts = list(sizes)
    while at < len(toks):
        n = min(cuts.pop(0) if cuts else len(toks), len(toks) - at)
        last = at + n == len(toks)
        tr.add([{"id": name, "tokens": toks[at:at + n], "want": list(range(n))}], [name] if last else [],
               [(rid, p) for p in range(at, at + n)])
        at += n


# ---------------------------------------------------------------------------
# One parallel layer whose attention makes ONE key stand out: the token NEEDLE gets a key along a
# feature that rotation leaves alone and that only the token PROBE asks for, and a value that moves
# the logits; the recurrent branch is silent.  Whether the probe finds the needle -- hundreds of
# positions back, across page borders, after decoding -- then decides the probe's logits.
NEEDLE, PROBE = 3, 5


def needle_model(heads=2, kv=1, dim=16, width=32, vocab=40, scale=1.0, rot_dims=8, taps=2):
    g = torch.Generator().manual_seed(7 * dim + heads)
    bf = torch.bfloat16
    rnd = lambda *shape: 0.02 * torch.randn(*shape, generator=g)
    E = 0.05 * torch.randn(vocab, width, generator=g)
    E[:, :2] = 0
    E[NEEDLE], E[PROBE] = 0, 0
    E[NEEDLE, 0], E[PROBE, 1] = 2.0, 2.0
    q, k, v = rnd(heads * dim, width), rnd(kv * dim, width), rnd(kv * dim, width)
    o = 0.05 * torch.randn(width, heads * dim, generator=g)
    f = rot_dims                                         # the first feature of a head that is not rotated
    for h in range(heads):
        q[h * dim + f] = 0
        q[h * dim + f, 1] = 4.0                          # the probe alone asks along that feature of every head
        o[0, h * dim + 1] = 1.0
    for h in range(kv):
        k[h * dim + f] = 0
        k[h * dim + f, 0] = 4.0                          # the needle alone answers there
        v[h * dim + 1, 0] = 2.0                          # and its value moves feature 0 of the residual: the needle's own logit
    ident = torch.zeros(1, taps)
    ident[0, -1] = 1.0                                   # a convolution that passes the current token through
    W = 16
    w = {"embed": E.to(bf)}
    for name, alpha in (("final.norm", 1.0), ("l0.norm1", 1.0), ("l0.norm1b", 1.0)):
        w[name], w[name + ".b"], w[name + ".alpha"] = torch.ones(width).to(bf), torch.zeros(width).to(bf), torch.tensor(alpha).to(bf)
    p = "l0.mix.left"
    w.update({f"{p}.q": q.to(bf), f"{p}.k": k.to(bf), f"{p}.v": v.to(bf), f"{p}.o": o.to(bf),
              f"{p}.q.b": torch.zeros(heads * dim).to(bf), f"{p}.k.b": torch.zeros(kv * dim).to(bf),
              f"{p}.v.b": torch.zeros(kv * dim).to(bf),
              f"{p}.q.conv": ident.repeat(heads * dim, 1).to(bf), f"{p}.k.conv": ident.repeat(kv * dim, 1).to(bf),
              f"{p}.v.conv": ident.repeat(kv * dim, 1).to(bf)})
    p = "l0.mix.right"
    w.update({f"{p}.y": rnd(W, width).to(bf), f"{p}.y.b": torch.zeros(W).to(bf), f"{p}.x": rnd(W, width).to(bf),
              f"{p}.x.b": torch.zeros(W).to(bf), f"{p}.conv": ident.repeat(W, 1).to(bf),
              f"{p}.conv.b": torch.zeros(W).to(bf), f"{p}.ra": torch.zeros(1, W, W).to(bf),
              f"{p}.ra.b": torch.zeros(1, W).to(bf), f"{p}.ri": torch.zeros(1, W, W).to(bf),
              f"{p}.ri.b": torch.zeros(1, W).to(bf), f"{p}.lam": torch.zeros(W).to(bf),
              f"{p}.o": torch.zeros(width, W).to(bf)})
    cfg = {"architecture": "Samulorn", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
           "embedding": {"scale": 1.0},
           "layers": [parallel_layer(heads, kv, dim, dim, taps, scale, {"base": 1e4, "dims": rot_dims}, W, 1, taps,
                                     1.0, 1.0, None)]}
    return cfg, w


def needle_tokens(n: int, needle_at: int, probes: List[int], vocab=40, seed=0) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    toks = torch.randint(8, vocab, (n,), generator=g).tolist()
    toks[needle_at] = NEEDLE
    for p in probes:
        toks[p] = PROBE
    return toks
