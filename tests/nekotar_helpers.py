"""Shared pieces of the Nekotar tests: small configurations that differ from each other in every
size and option, random weights by checkpoint name, and crafted one-layer models in which ONE
key stands out, so that a mask that is one position off, a lost far key or a latent row read
from the wrong place shows as a large error."""
from __future__ import annotations

import copy
from typing import Dict, List, Optional

import torch

from plain_nekotar import plain_forward


def _mlp(ff):
    return None if ff is None else {"kind": "dense", "ff": ff}


def wkv_layer(heads, dim, ff):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim}, "mlp": _mlp(ff)}


def latent_layer(heads, dim, rot_dim, vdim, rank, scale, base, ff, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": _mlp(ff)}


def window_layer(heads, kv, dim, vdim, scale, size, keep, base, dims, ff):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale,
                      "mask": {"size": size, "keep_first": keep}, "rot": {"base": base, "dims": dims}},
            "mlp": _mlp(ff)}


# three residual copies; every mixer; a latent layer that reads another's rows with fewer heads and
# other head sizes; rotation of half a head; wkv layers with and without a feed-forward
NEKO_A = {
    "architecture": "Nekotar", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "residual_mult": 0.7,
    "streams": 3,
    "layers": [wkv_layer(3, 16, 96),
               latent_layer(4, 16, 8, 24, 40, 0.2, 1e4, None),
               window_layer(4, 2, 16, 32, 0.3, 24, 5, 5e5, 8, 80),
               latent_layer(2, 8, 8, 16, 40, 0.3, 1e4, 64, kv_from=1),
               wkv_layer(2, 32, None)],
}
# ONE residual copy and factor 1 (the plain pre-norm sum), more kept positions than the window is
# long, head size 64 rotated in full, one wkv head, a latent row of 80 features
NEKO_B = {
    "architecture": "Nekotar", "vocab": 300, "width": 96, "norm": {"eps": 1e-6}, "residual_mult": 1.0,
    "streams": 1,
    "layers": [window_layer(6, 3, 64, 64, 0.11, 100, 130, 1e6, 64, 128),
               wkv_layer(1, 64, 64),
               latent_layer(3, 32, 16, 32, 64, 0.15, 2e4, None)],
}
# a width that is no multiple of 8 (products on the FMA kernel), two copies, key sizes 20 and 24, a
# latent row of 24 features with a rotated part of 4, a window of 7 after 3 kept positions, one
# kept position, value heads wider than key heads
NEKO_C = {
    "architecture": "Nekotar", "vocab": 130, "width": 100, "norm": {"eps": 1e-5}, "residual_mult": 0.25,
    "streams": 2,
    "layers": [latent_layer(5, 24, 4, 8, 20, 0.2, 1e4, None),
               window_layer(3, 1, 8, 8, 0.35, 7, 3, 1e4, 8, 50),
               wkv_layer(2, 20, 30),
               window_layer(2, 2, 24, 40, 0.2, 64, 1, 1e6, 12, None)],
}
# the inner size of every wkv layer's decay projection (the checkpoint's tensors give it), per layer
DECAY_RANKS = {"neko_a": {0: 8, 4: 4}, "neko_b": {1: 16}, "neko_c": {2: 3}}
CONFIGS = {"neko_a": (NEKO_A, 21), "neko_b": (NEKO_B, 32), "neko_c": (NEKO_C, 23)}

# Largest logit error relative to the request's largest logit.
# (A wkv head is divided by its own root mean square: where a head's output nearly cancels, its
# rounding error comes out at full size, so the 32-bit bound is wider than rounding alone.)
TOL = {"float32": 1e-4, "bfloat16": 6e-2, "float16": 8e-3}


def make_weights(cfg: dict, seed: int, dtype=torch.bfloat16, decay_ranks: Optional[Dict[int, int]] = None
                 ) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    D, V, s = cfg["width"], cfg["vocab"], cfg["streams"]
    mat = lambda r, c, std: (std * torch.randn(r, c, generator=g)).to(dtype)
    vec = lambda n, std: (std * torch.randn(n, generator=g)).to(dtype)
    ones = lambda n: (1.0 + 0.1 * torch.randn(n, generator=g)).to(dtype)
    w = {"embed": mat(V, D, 1.0), "embed.norm": ones(D), "final.norm": ones(D), "head": mat(V, D, 0.3)}
    a = D ** -0.5

    def copies(p):
        w[f"{p}.in"] = (1.0 / s + 0.2 * torch.randn(s, generator=g)).to(dtype)
        w[f"{p}.out"] = ones(s)
        w[f"{p}.mix"] = (torch.eye(s) + 0.15 * torch.randn(s, s, generator=g)).to(dtype)

    for i, layer in enumerate(cfg["layers"]):
        p, m, q = f"l{i}", layer["mixer"], f"l{i}.mix"
        w[f"{p}.norm1"] = ones(D)
        copies(f"{p}.hc1")
        if layer["type"] == "wkv":
            H, d = m["heads"], m["dim"]
            R = (decay_ranks or {}).get(i, 8)
            for name in "rkvgw":
                w[f"{q}.mu.{name}"] = torch.rand(D, generator=g).to(dtype)
            for name, std in (("r", 1.5), ("k", 1.5), ("v", 2.0), ("g", 2.0)):
                w[f"{q}.{name}"] = mat(H * d, D, std * a)
            w[f"{q}.w1"] = mat(R, D, 2.0 * a)
            w[f"{q}.w2"] = mat(H * d, R, R ** -0.5)
            # decays from nearly 1 (a state that remembers hundreds of tokens) down to a few tokens
            w[f"{q}.w0"] = (-6.0 + 6.5 * torch.rand(H * d, generator=g)).to(dtype)
            w[f"{q}.u"] = mat(H, d, 0.5)
            w[f"{q}.norm"] = ones(H * d)
            w[f"{q}.o"] = mat(D, H * d, 2.0 * (H * d) ** -0.5)
        elif layer["type"] == "latent_attention":
            H, d, rd, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            w[f"{q}.q"] = mat(H * (d + rd), D, 2.0 * a)
            if m.get("kv_from") is None:
                w[f"{q}.dkv"] = mat(R + rd, D, 2.0 * a)
                w[f"{q}.dkv.norm"] = ones(R)
            w[f"{q}.uk"] = mat(H * d, R, 2.0 * R ** -0.5)
            w[f"{q}.uv"] = mat(H * dv, R, 2.0 * R ** -0.5)
            w[f"{q}.g"] = mat(H * dv, D, 2.0 * a)
            w[f"{q}.o"] = mat(D, H * dv, 2.0 * (H * dv) ** -0.5)
        else:
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for name, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                w[f"{q}.{name}"] = mat(rows, D, 2.0 * a)
                w[f"{q}.{name}.b"] = vec(rows, 0.5)
            w[f"{q}.g"] = mat(H * dv, D, 2.0 * a)
            w[f"{q}.o"] = mat(D, H * dv, 2.0 * (H * dv) ** -0.5)
        if layer["mlp"]:
            ff = layer["mlp"]["ff"]
            w[f"{p}.norm2"] = ones(D)
            copies(f"{p}.hc2")
            w[f"{p}.mlp.up"] = mat(ff, D, 1.5 * a)
            w[f"{p}.mlp.down"] = mat(D, ff, 2.0 * ff ** -0.5)
    return w


def weights_of(name: str, dtype=torch.bfloat16):
    cfg, seed = CONFIGS[name]
    return make_weights(cfg, seed, dtype, DECAY_RANKS[name])


def random_tokens(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def references(cfg, w, reqs) -> Dict[str, torch.Tensor]:
    return {rid: plain_forward(cfg, w, toks) for rid, toks in reqs.items()}


def plain_generate_greedy(cfg, w, prompt: List[int], n_new: int) -> List[int]:
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(plain_forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]


# ---------------------------------------------------------------------------
# One layer whose weights make ONE key stand out: the token NEEDLE gets a key along a feature
# that rotation leaves alone and that only the token PROBE asks for, and a value that moves the
# logits.  Whether the needle is visible then decides the probe's logits.  (The embedding is
# normed, so ordinary tokens have features of size one; features 0 and 1 belong to the needle
# and the probe alone.)
NEEDLE, PROBE = 3, 5


def needle_model(kind: str, size: int = 0, keep: int = 0, heads=2, kv=1, dim=16, width=32, vocab=40,
                 scale=0.5, rot_dims=8, streams=2, rank=16):
    """``kind``: "attention" (a window of ``size`` after ``keep`` kept positions), "latent" (causal
    latent attention) or "shared_latent" (a silent latent layer, then one that reads its rows)."""
    g = torch.Generator().manual_seed(size * 131 + keep * 7 + dim)
    bf = torch.bfloat16
    rnd = lambda *shape: 0.02 * torch.randn(*shape, generator=g)
    E = 0.05 * torch.randn(vocab, width, generator=g)
    E[:, :2] = 0
    E[NEEDLE] = 0
    E[NEEDLE, 0] = 4.0
    E[PROBE] = 0
    E[PROBE, 1] = 4.0
    w = {"embed": E.to(bf), "embed.norm": torch.ones(width).to(bf), "final.norm": torch.ones(width).to(bf),
         "head": (0.5 * torch.randn(vocab, width, generator=g)).to(bf)}

    def copies(p, silent=False):
        w[f"{p}.in"] = torch.tensor([0.6, 0.5, 0.3, 0.2][:streams]).to(bf)
        w[f"{p}.out"] = torch.tensor([1.0, 0.5, -0.5, 0.25][:streams]).to(bf)
        mix = torch.eye(streams) if silent else torch.eye(streams) + 0.1 * torch.randn(streams, streams, generator=g)
        w[f"{p}.mix"] = mix.to(bf)

    if kind == "attention":
        layers = [window_layer(heads, kv, dim, dim, scale, size, keep, 1e4, rot_dims, None)]
        p, f = "l0.mix", rot_dims                     # f: the first feature of a head that is not rotated
        q, k, v = rnd(heads * dim, width), rnd(kv * dim, width), rnd(kv * dim, width)
        o = 0.05 * torch.randn(width, heads * dim, generator=g)
        for h in range(heads):
            q[h * dim + f] = 0
            q[h * dim + f, 1] = 1.0                    # the probe alone asks along that feature of every head
            o[2, h * dim + 1] = 1.0
        for h in range(kv):
            k[h * dim + f] = 0
            k[h * dim + f, 0] = 1.0                    # the needle alone answers there
            v[h * dim + 1, 0] = 1.0                    # and its value moves feature 2 of the residual
        w.update({"l0.norm1": torch.ones(width).to(bf), f"{p}.q": q.to(bf), f"{p}.k": k.to(bf), f"{p}.v": v.to(bf),
                  f"{p}.q.b": (0.05 * torch.randn(heads * dim, generator=g)).to(bf),
                  f"{p}.k.b": (0.05 * torch.randn(kv * dim, generator=g)).to(bf),
                  f"{p}.v.b": (0.05 * torch.randn(kv * dim, generator=g)).to(bf),
                  f"{p}.g": torch.zeros(heads * dim, width).to(bf), f"{p}.o": o.to(bf)})
        copies("l0.hc1")
    else:
        rd, vdim = rot_dims, dim
        own = latent_layer(heads, dim, rd, vdim, rank, scale, 1e4, None)
        layers = [own] if kind == "latent" else [own, latent_layer(heads, dim, rd, vdim, rank, scale, 1e4, None, kv_from=0)]
        dkv = rnd(rank + rd, width)
        dkv[0] = 0
        dkv[0, 0] = 3.0                                # the needle alone fills the latent's first feature
        for i in range(len(layers)):
            p = f"l{i}.mix"
            reads = i == len(layers) - 1               # the last layer looks for the needle; one before it is silent
            q, uk, uv = rnd(heads * (dim + rd), width), rnd(heads * dim, rank), rnd(heads * vdim, rank)
            o = 0.05 * torch.randn(width, heads * vdim, generator=g) if reads else torch.zeros(width, heads * vdim)
            for h in range(heads):
                q[h * (dim + rd)] = 0
                q[h * (dim + rd), 1] = 1.0             # unrotated query feature 0: the probe
                uk[h * dim] = 0
                uk[h * dim, 0] = 1.0                   # unrotated key feature 0: the latent's first feature
                uv[h * vdim + 1, 0] = 1.0
                if reads:
                    o[2, h * vdim + 1] = 1.0
            w.update({f"l{i}.norm1": torch.ones(width).to(bf), f"{p}.q": q.to(bf), f"{p}.uk": uk.to(bf),
                      f"{p}.uv": uv.to(bf), f"{p}.g": torch.zeros(heads * vdim, width).to(bf), f"{p}.o": o.to(bf)})
            if i == 0:
                w.update({f"{p}.dkv": dkv.to(bf), f"{p}.dkv.norm": torch.ones(rank).to(bf)})
            copies(f"l{i}.hc1", silent=not reads)
    cfg = {"architecture": "Nekotar", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
           "residual_mult": 0.5, "streams": streams, "layers": layers}
    return cfg, w


def needle_tokens(n: int, needle_at: int, probes: List[int], vocab=40, seed=0) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    toks = torch.randint(8, vocab, (n,), generator=g).tolist()
    toks[needle_at] = NEEDLE
    for p in probes:
        toks[p] = PROBE
    return toks


def with_mask(cfg: dict, **mask) -> dict:
    """The one-layer configuration with other mask numbers (what a library that is one off computes)."""
    out = copy.deepcopy(cfg)
    out["layers"][0]["mixer"]["mask"].update(mask)
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
