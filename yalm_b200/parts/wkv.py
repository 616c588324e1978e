"""A recurrence with a decay per key channel and a bonus for the current token ("wkv", the
time mixing of the RWKV family), per head with key size dk and value size dv:

    h'_t = h_(t-1)   (zero before a sequence's first token)
    x_s  = h + (h' - h) mu_s                       for s in r, k, v, g, w
    r, k = Wr x_r, Wk x_k  [H, dk];   v = Wv x_v  [H, dv];   gate = silu(Wg x_g)
    w    = exp(-exp(W2 tanh(W1 x_w) + w0))         a decay per head and key channel
    o_t  = (S_(t-1) + diag(u) k_t v_t^T)^T r_t,    S_t = diag(w_t) S_(t-1) + k_t v_t^T

Each head's o_t is divided by its root mean square, the heads are concatenated, multiplied by a
weight per feature and by the gate, and projected by Wo.  Two fixed-size per-sequence cache needs:
the state S (float32 [H, dk, dv]) and the previous token's input (float32 [width]).  Mixtures are
rounded to the compute type as the products' inputs; decays, state, output norm and gate are
32-bit.
"""
from __future__ import annotations

import torch

from ..cache import CacheNeed
from ..csrc import ops
from ..weights import TensorNeed
from .base import register_mixer
from .linear import matmul_act, matmul_partials

MIXES = ("r", "k", "v", "g", "w")


@register_mixer("wkv_time_mix")
class WkvTimeMix:
    def __init__(self, params: dict, rt):
        self.rt = rt
        self.D = int(params["hidden_size"])
        self.H = int(params["num_heads"])
        self.dk = int(params["key_dim"])
        self.dv = int(params.get("value_dim") or self.dk)
        self.rank = int(params["decay_rank"])
        self.eps = float(params["eps"])
        if min(self.H, self.dk, self.dv, self.rank) <= 0 or self.dk > 256:
            raise ValueError(f"wkv_time_mix: heads {self.H}, key size {self.dk} (up to 256), value size "
                             f"{self.dv}, decay rank {self.rank}")
        self.mu = self.w = self.w0 = self.bonus = self.norm = None

    def tensor_needs(self):
        H, dk, dv, D, R = self.H, self.dk, self.dv, self.D, self.rank
        needs = {f"mu.{s}": TensorNeed((D,), init="fraction") for s in MIXES}
        needs.update({"r": TensorNeed((H * dk, D)), "k": TensorNeed((H * dk, D)), "v": TensorNeed((H * dv, D)),
                      "g": TensorNeed((H * dv, D)), "w1": TensorNeed((R, D)), "w2": TensorNeed((H * dk, R)),
                      "w0": TensorNeed((H * dk,), init="around_zero"), "u": TensorNeed((H, dk), init="around_zero"),
                      "norm": TensorNeed((H * dv,), init="ones"), "o": TensorNeed((D, H * dv))})
        return needs

    def bind(self, tensors) -> None:
        rt = self.rt
        self.mu = torch.stack([rt.vector(tensors[f"mu.{s}"]) for s in MIXES]).contiguous()
        self.w = {k: rt.matrix(tensors[k]) for k in ("r", "k", "v", "g", "w1", "w2", "o")}
        self.w0 = rt.vector(tensors["w0"])
        self.bonus = rt.vector(tensors["u"]).reshape(-1).contiguous()
        self.norm = rt.vector(tensors["norm"])

    def cache_need(self):
        return {"state": CacheNeed("state", state_shape=(self.H, self.dk, self.dv), state_dtype=torch.float32),
                "previous": CacheNeed("state", state_shape=(self.D,), state_dtype=torch.float32)}

    def cache_read_bytes(self, contexts, element_size: int) -> int:
        return 2 * len(contexts) * (self.H * self.dk * self.dv + self.D) * 4      # read and written

    def flops(self, q_lens, past) -> float:
        n = sum(q_lens)
        H, dk, dv, D, R = self.H, self.dk, self.dv, self.D, self.rank
        return 2.0 * n * ((2 * dk + 2 * dv) * H * D + R * D + H * dk * R + D * H * dv) + 6.0 * n * H * dk * dv

    def forward(self, h, batch, stream, view, shared: bool = False):
        if shared:
            raise RuntimeError("a recurrent state cannot be read by another run entry")
        rt, H, dk, dv = self.rt, self.H, self.dk, self.dv
        n = batch.n_tokens
        state, prev = view["state"].state, view["previous"].state
        mixed = rt.buffer("wkv_mixed", (len(MIXES), n, self.D), rt.dtype)
        ops.token_shift(h, prev, self.mu, mixed, batch)
        proj = {s: matmul_partials(rt, mixed[i], self.w[s], f"wkv_{s}") for i, s in enumerate(MIXES[:4])}
        low_act = rt.buffer("wkv_w1_act", (n, self.rank), rt.dtype)
        matmul_act(rt, mixed[4], self.w["w1"], low_act, ops.TANH, "wkv_w1")
        z = matmul_partials(rt, low_act, self.w["w2"], "wkv_w2")
        act = rt.buffer("wkv_act", (n, 3 * H * dk + H * dv), torch.float32)
        gate = rt.buffer("wkv_gate", (n, H * dv), torch.float32)
        o = rt.buffer("wkv_o", (n, H * dv), torch.float32)
        ops.wkv(proj["r"], proj["k"], proj["v"], proj["g"], z, self.w0, self.bonus, act, gate, h, prev,
                batch, state, o, H, dk, dv)
        on = rt.buffer("wkv_normed", (n, H * dv), rt.dtype)
        ops.wkv_out(o, self.norm, gate, on, H, dv, self.eps)
        stream.add_linear(on, self.w["o"])
        return None
