"""A plain, slow statement of the Samulorn decoder in torch on the CPU, one function per
mechanism, written from the design's equations and sharing no code with the library.  It keeps
every sequence's state in a dict so that a prompt can be fed in pieces.

Notation: T tokens of one sequence, width D.  Weights are [out, in] and applied as W x.

    dyt(x)            = tanh(alpha x) w + b                         (the model's norm: no mean, no variance)
    layer             : x += dyt1b(mixer(dyt1(x)));  x += dyt2b(ff(dyt2(x)));  x += side(x, token)
    side              : g = gelu(Wg x) * E_side[token, part of the layer];  y = Wp g;
                        x += y / sqrt(mean(y^2) + eps) * w
    channel_delta     : q, k, v = silu(conv(W. h));  q, k unit vectors per head, q / sqrt(dim);
                        beta = sigmoid(Wb h);  decay = exp(-exp(A) softplus(Wa2 Wa1 h + dt)) per key channel;
                        S <- decay S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
                        o / rms(o) * w * sigmoid(Wg2 Wg1 h);  Wo
    parallel          : left_scale * attention(h) + right_scale * rglru(h)
    attention (left)  : q, k, v = conv(W. h + b);  rotate the first `dims` of q, k in pairs (2i, 2i+1);
                        q, k over their root mean square per head;  softmax(scale q.k) v, causal;  Wo
    rglru (right)     : y = gelu(Wy h + by);  u = conv(Wx h + bx) + bc;  r, i = sigmoid(block-diagonal(u) + b);
                        a = exp(-8 r softplus(lam));  S <- a S + sqrt(1 - a^2) i u;  Wo (S y)
    experts           : s = sigmoid(Wr h);  choice = s + correction;  groups by the sum of their two best
                        choices;  top experts of the kept groups;  weights s / (sum + 1e-20) * scale
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def dyt(x, alpha, w, b):
    return torch.tanh(alpha * x) * w + b


def over_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def short_conv(u, w, before):
    """u [T, C]; w [C, taps] with the last column for the current token; ``before`` [taps - 1, C], the
    inputs that came before u (zeros for a new sequence).  Returns (y [T, C], the new ``before``)."""
    taps = w.shape[1]
    full = torch.cat([before, u], 0)                       # [taps - 1 + T, C]
    T = u.shape[0]
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + full[j:j + T] * w[:, j]
    return y, full[full.shape[0] - (taps - 1):]


def rotary_frequencies(dims: int, base: float, scaling: Optional[dict]):
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling:
            factor, low, high = float(scaling["factor"]), float(scaling["low"]), float(scaling["high"])
            orig = float(scaling["original"])
            wave = 2.0 * math.pi / f
            if wave < orig / high:
                pass
            elif wave > orig / low:
                f = f / factor
            else:
                s = (orig / wave - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64)


def rotate_neighbours(x, positions, freqs):
    """x [T, heads, size]; the first 2 * len(freqs) features of every head are rotated in pairs
    (2i, 2i + 1) by positions[t] * freqs[i]."""
    dims = 2 * len(freqs)
    ang = (positions.to(torch.float32)[:, None] * freqs.to(torch.float32)[None, :])      # [T, dims/2]
    c, s = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def causal_attention(q, k, v, past_k, past_v, scale):
    """q [T, H, d], k [T, G, d], v [T, G, dv] of this piece; past_k / past_v the earlier ones.
    Returns (o [T, H, dv], all keys, all values)."""
    K = torch.cat([past_k, k], 0)
    V = torch.cat([past_v, v], 0)
    T, H, _ = q.shape
    G = k.shape[1]
    P = past_k.shape[0]
    o = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ K[:, g].T) * scale                                  # [T, P + T]
        idx = torch.arange(P + T)[None, :]
        s = s.masked_fill(idx > (torch.arange(T)[:, None] + P), float("-inf"))
        o[:, h] = torch.softmax(s, -1) @ V[:, g]
    return o, K, V


def delta_rule(q, k, v, beta, decay, S):
    """One head over T tokens: q, k, decay [T, dk]; v [T, dv]; beta [T]; S [dk, dv] (changed in place)."""
    out = []
    for t in range(q.shape[0]):
        S.mul_(decay[t][:, None])
        u = beta[t] * (v[t] - S.T @ k[t])
        S.add_(torch.outer(k[t], u))
        out.append(S.T @ q[t])
    return torch.stack(out)


def route(z, correction, groups: int, keep: int, top: int, scale: float):
    """z [E] router logits of one token -> (chosen experts, their weights, margin): the margin is the
    smallest gap between something chosen and the best thing not chosen (groups, then experts); a
    16-bit computation may rightly decide a call that close the other way."""
    s = torch.sigmoid(z)
    choice = s + correction
    E = z.numel()
    per = E // groups
    gs = choice.view(groups, per).topk(min(2, per), -1).values.sum(-1)
    order = gs.argsort(descending=True)
    kept = order[:keep]
    margin = float(gs[order[keep - 1]] - gs[order[keep]]) if keep < groups else float("inf")
    mask = torch.full((groups, per), float("-inf"), dtype=z.dtype)
    mask[kept] = 0.0
    cand = choice + mask.view(-1)
    ranked = cand.argsort(descending=True)
    chosen = ranked[:top]
    if top < keep * per:
        margin = min(margin, float(cand[ranked[top - 1]] - cand[ranked[top]]))
    w = s[chosen]
    return chosen, w / (w.sum() + 1e-20) * scale, margin


class PlainSamulorn:
    def __init__(self, config: dict, tensors: Dict[str, torch.Tensor], dtype=torch.float32):
        self.c = config
        self.dt = dtype
        self.w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
        self.eps = float(config["norm"]["eps"])
        self.D = int(config["width"])
        n = len(config["layers"])
        loop = config.get("loop") or None
        if loop and int(loop.get("times", 1)) > 1:
            a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
            self.runs = list(range(a)) + list(range(a, b)) * times + list(range(b, n))
        else:
            self.runs = list(range(n))
        self.taps = None                                   # called as taps(run index, x [T, D]) after a layer run
        self.margins: List[float] = []                     # of every routing decision made, in order

    def new_state(self) -> dict:
        return {"pos": 0, "runs": [dict() for _ in self.runs]}

    # -- pieces ----------------------------------------------------------------------------------------
    def _norm(self, name, x):
        w = self.w
        return dyt(x, w[name + ".alpha"], w[name], w[name + ".b"])

    def _conv(self, st, key, u, weight):
        taps = weight.shape[1]
        before = st.get(key)
        if before is None:
            before = torch.zeros(taps - 1, u.shape[1], dtype=u.dtype)
        y, st[key] = short_conv(u, weight, before)
        return y

    def _channel_delta(self, p, m, h, st):
        w = self.w
        H, G, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
        T = h.shape[0]
        q = F.silu(self._conv(st, "q", h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, dk)
        k = F.silu(self._conv(st, "k", h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, dk)
        v = F.silu(self._conv(st, "v", h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, dv)
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        beta = torch.sigmoid(h @ w[p + "b"].T)                                       # [T, H]
        a = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]
        decay = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * F.softplus(a).view(T, H, dk))
        S = st.setdefault("S", torch.zeros(H, dk, dv, dtype=h.dtype))
        o = torch.stack([delta_rule(q[:, hh // (H // G)], k[:, hh // (H // G)], v[:, hh], beta[:, hh],
                                    decay[:, hh], S[hh]) for hh in range(H)], 1)     # [T, H, dv]
        gate = torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).view(T, H, dv)
        o = over_rms(o, self.eps) * w[p + "norm"] * gate
        return o.reshape(T, H * dv) @ w[p + "o"].T

    def _left(self, p, m, h, st, pos0):
        w = self.w
        H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
        T = h.shape[0]
        q = self._conv(st, "lq", h @ w[p + "q"].T + w[p + "q.b"], w[p + "q.conv"]).view(T, H, d)
        k = self._conv(st, "lk", h @ w[p + "k"].T + w[p + "k.b"], w[p + "k.conv"]).view(T, G, d)
        v = self._conv(st, "lv", h @ w[p + "v"].T + w[p + "v.b"], w[p + "v.conv"]).view(T, G, dv)
        rot = m.get("rot") or None
        if rot and int(rot.get("dims", 0)) > 0:
            f = rotary_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
            positions = torch.arange(pos0, pos0 + T)
            q, k = rotate_neighbours(q, positions, f), rotate_neighbours(k, positions, f)
        q, k = over_rms(q, self.eps), over_rms(k, self.eps)
        pk = st.get("K", torch.zeros(0, G, d, dtype=h.dtype))
        pv = st.get("V", torch.zeros(0, G, dv, dtype=h.dtype))
        o, st["K"], st["V"] = causal_attention(q, k, v, pk, pv, float(m["scale"]))
        return o.reshape(T, H * dv) @ w[p + "o"].T

    def _right(self, p, m, h, st):
        w = self.w
        W, B = int(m["width"]), int(m["blocks"])
        T = h.shape[0]
        y = gelu_tanh(h @ w[p + "y"].T + w[p + "y.b"])
        u = self._conv(st, "ru", h @ w[p + "x"].T + w[p + "x.b"], w[p + "conv"]) + w[p + "conv.b"]
        ub = u.view(T, B, W // B)
        r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + "ra"]) + w[p + "ra.b"]).reshape(T, W)
        i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + "ri"]) + w[p + "ri.b"]).reshape(T, W)
        a = torch.exp(-8.0 * r * F.softplus(w[p + "lam"]))
        S = st.get("R", torch.zeros(W, dtype=h.dtype))
        out = []
        for t in range(T):
            S = a[t] * S + torch.sqrt(1.0 - a[t] * a[t]) * i[t] * u[t]
            out.append(S)
        st["R"] = S
        return (torch.stack(out) * y) @ w[p + "o"].T

    def _glu(self, p, h):
        w = self.w
        return (F.silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T

    def _experts(self, p, m, h):
        w = self.w
        r = m["router"]
        z = h @ w[p + "router"].T
        out = torch.zeros_like(h)
        for t in range(h.shape[0]):
            g = r.get("groups") or {"count": 1, "keep": 1}
            chosen, weights, margin = route(z[t], w[p + "correction"], int(g["count"]), int(g["keep"]),
                                            int(r["top"]), float(r.get("scale", 1.0)))
            self.margins.append(margin)
            for e, wt in zip(chosen.tolist(), weights):
                out[t] += wt * self._glu(f"{p}e{e}.", h[t:t + 1])[0]
        return out

    # -- the model -------------------------------------------------------------------------------------
    def forward(self, tokens: List[int], state: dict) -> torch.Tensor:
        """Feeds ``tokens`` as the sequence's next ones; returns logits [T, vocab]."""
        c, w = self.c, self.w
        tok = torch.tensor(tokens, dtype=torch.long)
        T = len(tokens)
        pos0 = state["pos"]
        x = w["embed"][tok] * float(c["embedding"]["scale"])
        sd = int(c["token_side"]["dim"]) if c.get("token_side") else 0
        for ri, li in enumerate(self.runs):
            L = c["layers"][li]
            st = state["runs"][ri]
            pre = f"l{li}."
            h = self._norm(pre + "norm1", x)
            if L["type"] == "channel_delta":
                y = self._channel_delta(pre + "mix.", L["mixer"], h, st)
            elif L["type"] == "parallel":
                m = L["mixer"]
                y = float(m["left_scale"]) * self._left(pre + "mix.left.", m["left"], h, st, pos0) \
                    + float(m["right_scale"]) * self._right(pre + "mix.right.", m["right"], h, st)
            else:
                raise ValueError(L["type"])
            x = x + self._norm(pre + "norm1b", y)
            mlp = L.get("mlp")
            if mlp:
                h = self._norm(pre + "norm2", x)
                y = self._glu(pre + "mlp.", h) if mlp["kind"] == "dense" else self._experts(pre + "mlp.", mlp, h)
                x = x + self._norm(pre + "norm2b", y)
            if sd:
                e = w["side.embed"][tok][:, li * sd:(li + 1) * sd]
                g = gelu_tanh(x @ w[pre + "side.gate"].T) * e
                y = g @ w[pre + "side.proj"].T
                x = x + over_rms(y, self.eps) * w[pre + "side.norm"]
            if self.taps is not None:
                self.taps(ri, x)
        state["pos"] = pos0 + T
        return self._norm("final.norm", x) @ w["embed"].T
