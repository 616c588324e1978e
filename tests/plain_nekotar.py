"""A plain, slow implementation of the Nekotar decoder for tests: whole sequences, no cache,
one function per mechanism, on the CPU.  It reads the raw ``config.json`` dictionary and
tensors by their checkpoint names and shares no code with the library under test.

The design in this file's notation (T tokens, width D, n(u) = u / sqrt(mean u^2 + eps)):

* embedding: x_t = n(E[tok_t]) * w_embed;
* s residual copies X_1 .. X_s, all equal to the embedding output.  A sublayer f with its read
  weights a [s], write weights b [s] and mixing matrix M [s, s] (from, to):
      u = sum_i a_i X_i;  y = f(n(u) * w);  X_j <- sum_i M_ij X_i + m b_j y   (all j from the old X)
  with m the model's residual factor.  A layer is a mixer sublayer and, where it has one, a
  feed-forward sublayer.  The model's output reads X_1 + .. + X_s;
* mixer "wkv": with h'_t = h_(t-1) (zero at t = 0), every one of r, k, v, g, w reads
  h + (h' - h) mu of its own; r, k, v = W h_mix per head, gate = silu(Wg h_g),
  decay d = exp(-exp(W2 tanh(W1 h_w) + w0)) per head and key channel; per head
      o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t,   S_t = diag(d_t) S_(t-1) + k_t v_t^T;
  every head's o over its root mean square, heads side by side, times a weight, times the
  gate, then Wo;
* mixer "latent_attention": q = Wq h, per head [dim | rot_dim]; Wdkv h = [c' | kr]; c = n(c') w_c;
  per head k = [Wuk c | rot(kr)], v = Wuv c, queries rotated on their last rot_dim features in
  neighbouring pairs; causal softmax(scale q.k); heads side by side times sigmoid(Wg h); Wo.  A
  layer with ``kv_from`` = j takes c and rot(kr) from layer j;
* mixer "attention": q, k, v with biases, grouped heads, the first ``rot.dims`` features of each
  head rotated in pairs (i, i + dims/2); query i sees key j <= i when i - j < size or
  j < keep_first; softmax(scale q.k); times sigmoid(Wg h); Wo;
* feed-forward: Wdown gelu_tanh(Wup h);
* output: n(sum_i X_i) w_final, head.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch


def plain_norm(u: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight.to(u.dtype)


def plain_embedding(w, cfg: dict, tokens: Sequence[int], dt) -> torch.Tensor:
    x = w["embed"].to(dt)[torch.tensor(list(tokens), dtype=torch.long)]
    return plain_norm(x, w["embed.norm"], float(cfg["norm"]["eps"]))


def plain_gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# ----------------------------------------------------------------------------- rotation
def plain_rotate(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int, neighbours: bool) -> torch.Tensor:
    """x [T, heads, size]: the first ``dims`` features of each head rotated by position * base^(-2i/dims)."""
    if not dims:
        return x
    i = torch.arange(dims // 2, dtype=torch.float64)
    ang = (positions.to(torch.float64)[:, None] * base ** (-2.0 * i / dims)).to(torch.float32)
    cos, sin = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    out = x.clone()
    if neighbours:
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = a * cos - b * sin
        out[..., 1:dims:2] = b * cos + a * sin
    else:
        a, b = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2] = a * cos - b * sin
        out[..., dims // 2:dims] = b * cos + a * sin
    return out


def plain_softmax_mix(q, k, v, scale: float, visible: torch.Tensor) -> torch.Tensor:
    """q [T, H, dk], k [T, H, dk], v [T, H, dv], visible [T, T] bool -> [T, H, dv]."""
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    s = s.masked_fill(~visible[None], float("-inf"))
    return torch.einsum("hij,jhd->ihd", torch.softmax(s, dim=-1), v)


def plain_kept_window_mask(T: int, size: int, keep_first: int) -> torch.Tensor:
    """[T, T] bool: query i sees key j <= i inside the last ``size`` positions or among the first ``keep_first``."""
    pos = torch.arange(T)
    i, j = pos[:, None], pos[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


# ----------------------------------------------------------------------------- mixers
def plain_window_attention(w, p: str, m: dict, h: torch.Tensor) -> torch.Tensor:
    T, dt = h.shape[0], h.dtype
    H, G, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    lin = lambda name: h @ w[f"{p}.{name}"].to(dt).T + w[f"{p}.{name}.b"].to(dt)
    q, k, v = lin("q").view(T, H, dk), lin("k").view(T, G, dk), lin("v").view(T, G, dv)
    pos = torch.arange(T)
    rot = m.get("rot")
    if rot:
        q = plain_rotate(q, pos, float(rot["base"]), int(rot["dims"]), neighbours=False)
        k = plain_rotate(k, pos, float(rot["base"]), int(rot["dims"]), neighbours=False)
    k = k.repeat_interleave(H // G, dim=1)
    v = v.repeat_interleave(H // G, dim=1)
    mask = m.get("mask")
    visible = plain_kept_window_mask(T, int(mask["size"]), int(mask.get("keep_first", 0))) if mask \
        else pos[None, :] <= pos[:, None]
    o = plain_softmax_mix(q, k, v, float(m["scale"]), visible).reshape(T, H * dv)
    o = o * torch.sigmoid(h @ w[f"{p}.g"].to(dt).T)
    return o @ w[f"{p}.o"].to(dt).T


def plain_latent(w, p: str, m: dict, h: torch.Tensor, eps: float):
    """The latent rows c [T, rank] and the rotated shared key part [T, rot_dim] of a layer that owns them."""
    dt = h.dtype
    rank, rd = int(m["kv_rank"]), int(m["rot_dim"])
    z = h @ w[f"{p}.dkv"].to(dt).T
    c = plain_norm(z[:, :rank], w[f"{p}.dkv.norm"], eps)
    kr = plain_rotate(z[:, None, rank:rank + rd], torch.arange(h.shape[0]), float(m["rot"]["base"]), rd,
                      neighbours=True)[:, 0]
    return c, kr


def plain_latent_attention(w, p: str, m: dict, h: torch.Tensor, c: torch.Tensor, kr: torch.Tensor) -> torch.Tensor:
    T, dt = h.shape[0], h.dtype
    H, dk, rd, dv = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"])
    q = (h @ w[f"{p}.q"].to(dt).T).view(T, H, dk + rd)
    q_rot = plain_rotate(q[..., dk:], torch.arange(T), float(m["rot"]["base"]), rd, neighbours=True)
    q = torch.cat([q[..., :dk], q_rot], -1)
    k_up = (c @ w[f"{p}.uk"].to(dt).T).view(T, H, dk)
    k = torch.cat([k_up, kr[:, None, :].expand(T, H, rd)], -1)
    v = (c @ w[f"{p}.uv"].to(dt).T).view(T, H, dv)
    pos = torch.arange(T)
    o = plain_softmax_mix(q, k, v, float(m["scale"]), pos[None, :] <= pos[:, None]).reshape(T, H * dv)
    o = o * torch.sigmoid(h @ w[f"{p}.g"].to(dt).T)
    return o @ w[f"{p}.o"].to(dt).T


def plain_wkv(w, p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    T, dt = h.shape[0], h.dtype
    H, d = int(m["heads"]), int(m["dim"])
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], 0)
    mix = lambda s: h + (prev - h) * w[f"{p}.mu.{s}"].to(dt)
    r = (mix("r") @ w[f"{p}.r"].to(dt).T).view(T, H, d)
    k = (mix("k") @ w[f"{p}.k"].to(dt).T).view(T, H, d)
    v = (mix("v") @ w[f"{p}.v"].to(dt).T).view(T, H, d)
    gate = torch.nn.functional.silu(mix("g") @ w[f"{p}.g"].to(dt).T)
    z = torch.tanh(mix("w") @ w[f"{p}.w1"].to(dt).T) @ w[f"{p}.w2"].to(dt).T + w[f"{p}.w0"].to(dt)
    decay = torch.exp(-torch.exp(z)).view(T, H, d)
    u = w[f"{p}.u"].to(dt)                                      # [H, d]
    S = torch.zeros(H, d, d, dtype=dt)
    o = torch.zeros(T, H, d, dtype=dt)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]                # [H, key, value]
        o[t] = torch.einsum("hkv,hk->hv", S + u[:, :, None] * kv, r[t])
        S = decay[t][:, :, None] * S + kv
    o = plain_norm(o, None, eps).reshape(T, H * d) * w[f"{p}.norm"].to(dt) * gate
    return o @ w[f"{p}.o"].to(dt).T


def plain_feed_forward(w, p: str, h: torch.Tensor) -> torch.Tensor:
    dt = h.dtype
    return plain_gelu_tanh(h @ w[f"{p}.up"].to(dt).T) @ w[f"{p}.down"].to(dt).T


# ----------------------------------------------------------------------------- residual copies
def plain_sublayer(w, p: str, X: torch.Tensor, norm_w: torch.Tensor, eps: float, m: float, f) -> torch.Tensor:
    """X [s, T, D] -> the new X: read with ``in``, write with ``mix`` [from, to] and ``out``."""
    dt = X.dtype
    a, b, M = w[f"{p}.in"].to(dt), w[f"{p}.out"].to(dt), w[f"{p}.mix"].to(dt)
    u = torch.einsum("s,std->td", a, X)
    y = f(plain_norm(u, norm_w, eps))
    return torch.einsum("sj,std->jtd", M, X) + m * b[:, None, None] * y[None]


def plain_forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], dtype=torch.float64,
                  layer_outputs: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  ``layer_outputs`` collects the sum of the residual
    copies after every layer."""
    eps, m, s = float(cfg["norm"]["eps"]), float(cfg["residual_mult"]), int(cfg["streams"])
    x = plain_embedding(w, cfg, tokens, dtype)
    X = x[None].repeat(s, 1, 1)
    latents = {}
    for i, layer in enumerate(cfg["layers"]):
        p, mx, kind = f"l{i}", layer["mixer"], layer["type"]
        if kind == "wkv":
            f = lambda h: plain_wkv(w, f"{p}.mix", mx, h, eps)
        elif kind == "attention":
            f = lambda h: plain_window_attention(w, f"{p}.mix", mx, h)
        elif kind == "latent_attention":
            def f(h):
                src = mx.get("kv_from")
                if src is None:
                    latents[i] = plain_latent(w, f"{p}.mix", mx, h, eps)
                    src = i
                return plain_latent_attention(w, f"{p}.mix", mx, h, *latents[int(src)])
        else:
            raise ValueError(kind)
        X = plain_sublayer(w, f"{p}.hc1", X, w[f"{p}.norm1"], eps, m, f)
        if layer.get("mlp"):
            X = plain_sublayer(w, f"{p}.hc2", X, w[f"{p}.norm2"], eps, m,
                               lambda h: plain_feed_forward(w, f"{p}.mlp", h))
        if layer_outputs is not None:
            layer_outputs.append(X.sum(0))
    x = plain_norm(X.sum(0), w["final.norm"], eps)
    return x @ w["head"].to(dtype).T
