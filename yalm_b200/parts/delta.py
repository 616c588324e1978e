"""The gated delta rule with a decay per key channel, per head with key size dk and value size dv:

    q, k, v = silu(conv(Wq h)), silu(conv(Wk h)), silu(conv(Wv h))     a short causal convolution over time
    q, k    <- unit vectors per head (x / sqrt(sum x^2 + 1e-6)),  q also times dk^-1/2
    beta    = sigmoid(Wb h)                                            one per head
    g       = exp(-exp(A_h) softplus(Wa2 (Wa1 h) + dt))                per head and key channel
    S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

so the read-out sees the current token's write.  q and k may have fewer heads than v (head h reads
q/k head h // (H / G)).  Each head's o is divided by its root mean square, multiplied by a weight per
value channel (shared by the heads) and by sigmoid(Wg2 (Wg1 h)), and projected by Wo.  Three
fixed-size cache needs per sequence: the state S (float32 [H, dk, dv]) and the convolution's last
taps - 1 inputs (float32 [taps - 1, 2 G dk + H dv]).  The six projections that read h are one product;
the two low-rank second halves are one product over a block-diagonal matrix.  Convolution, unit
vectors, gates, decay, state and output norm are 32-bit.
"""
from __future__ import annotations

import torch

from ..cache import CacheNeed
from ..csrc import ops
from ..weights import TensorNeed
from .base import register_mixer
from .linear import matmul_partials

UNIT_EPS = 1e-6          # the design's own: inside the root of the unit vectors


@register_mixer("gated_delta_rule")
class GatedDeltaRule:
    def __init__(self, params: dict, rt):
        self.rt = rt
        self.D = int(params["hidden_size"])
        self.H = int(params["num_heads"])
        self.G = int(params.get("num_kv_heads") or self.H)
        self.dk = int(params["key_dim"])
        self.dv = int(params.get("value_dim") or self.dk)
        self.taps = int(params["conv"])
        self.rank_a = int(params["decay_rank"])
        self.rank_g = int(params["gate_rank"])
        self.eps = float(params["eps"])
        if min(self.H, self.G, self.dk, self.dv, self.rank_a, self.rank_g) <= 0 or self.H % self.G \
                or self.dk > 256 or not 2 <= self.taps <= 8:
            raise ValueError(f"gated_delta_rule: heads {self.H} over {self.G} q/k heads, key size {self.dk} (up to "
                             f"256), value size {self.dv}, convolution of {self.taps} taps (2 to 8)")
        self.C = 2 * self.G * self.dk + self.H * self.dv          # convolved channels: q | k | v
        self.w_in = self.w_low = self.w_o = None
        self.conv_w = self.dt_bias = self.a_log = self.norm = None

    def tensor_needs(self):
        H, G, dk, dv, D = self.H, self.G, self.dk, self.dv, self.D
        return {"q": TensorNeed((G * dk, D)), "k": TensorNeed((G * dk, D)), "v": TensorNeed((H * dv, D)),
                "q.conv": TensorNeed((G * dk, self.taps)), "k.conv": TensorNeed((G * dk, self.taps)),
                "v.conv": TensorNeed((H * dv, self.taps)), "b": TensorNeed((H, D)),
                "A_log": TensorNeed((H,), init="around_zero"),
                "a1": TensorNeed((self.rank_a, D)), "a2": TensorNeed((H * dk, self.rank_a)),
                "dt_bias": TensorNeed((H * dk,), init="around_zero"),
                "g1": TensorNeed((self.rank_g, D)), "g2": TensorNeed((H * dv, self.rank_g)),
                "norm": TensorNeed((dv,), init="ones"), "o": TensorNeed((D, H * dv))}

    def bind(self, tensors) -> None:
        rt = self.rt
        first = [tensors[k] for k in ("q", "k", "v", "b", "a1", "g1")]
        second = [tensors["a2"], tensors["g2"]]
        if any(p.dtype == torch.float32 for p in first + second):
            first, second = [p.to(torch.float32) for p in first], [p.to(torch.float32) for p in second]
        # [a2 0; 0 g2]: both second halves in one product over the row [a1 h | g1 h]; the row is
        # padded with zero columns to a multiple of 8 (the tensor-core product's row pitch)
        ra, rg = self.rank_a, self.rank_g
        self.n_low = -(-(ra + rg) // 8) * 8
        low = torch.zeros((self.H * self.dk + self.H * self.dv, self.n_low), dtype=second[0].dtype)
        low[:self.H * self.dk, :ra] = second[0]
        low[self.H * self.dk:, ra:ra + rg] = second[1]
        self.w_low = rt.matrix(low)
        if self.n_low != ra + rg:                       # the zero columns' inputs: rows of zeros in the first product
            first.append(torch.zeros((self.n_low - ra - rg, self.D), dtype=first[0].dtype))
        self.w_in = rt.matrix(torch.cat(first, 0))
        self.w_o = rt.matrix(tensors["o"])
        self.conv_w = torch.cat([rt.vector(tensors[k]) for k in ("q.conv", "k.conv", "v.conv")], 0).contiguous()
        self.dt_bias = rt.vector(tensors["dt_bias"])
        self.a_log = rt.vector(tensors["A_log"])
        self.norm = rt.vector(tensors["norm"]).repeat(self.H).contiguous()

    def cache_need(self):
        return {"state": CacheNeed("state", state_shape=(self.H, self.dk, self.dv), state_dtype=torch.float32),
                "conv": CacheNeed("state", state_shape=(self.taps - 1, self.C), state_dtype=torch.float32)}

    def cache_read_bytes(self, contexts, element_size: int) -> int:
        return 2 * len(contexts) * (self.H * self.dk * self.dv + (self.taps - 1) * self.C) * 4

    def flops(self, q_lens, past) -> float:
        n = sum(q_lens)
        H, dk, dv, D = self.H, self.dk, self.dv, self.D
        return 2.0 * n * ((self.C + H + self.rank_a + self.rank_g) * D + (H * dk) * self.rank_a
                          + (H * dv) * self.rank_g + D * H * dv) + 8.0 * n * H * dk * dv

    def forward(self, h, batch, stream, view, shared: bool = False):
        if shared:
            raise RuntimeError("a recurrent state cannot be read by another run entry")
        rt, H, G, dk, dv, C = self.rt, self.H, self.G, self.dk, self.dv, self.C
        n = batch.n_tokens
        proj, S = matmul_partials(rt, h, self.w_in, "delta_in")
        act = rt.buffer("delta_act", (n, ops.delta_row(H, G, dk, dv)), torch.float32)
        ops.short_conv(proj, S, 0, C, self.conv_w, view["conv"].state, batch, out32=act, silu=True)
        low = rt.buffer("delta_low", (n, self.n_low), rt.dtype)
        ops.delta_prep(act, proj, S, C, C + H, self.n_low, low, H, G, dk, dv)
        z, Sz = matmul_partials(rt, low, self.w_low, "delta_low_out")
        gate = rt.buffer("delta_gate", (n, H * dv), torch.float32)
        o = rt.buffer("delta_o", (n, H * dv), torch.float32)
        ops.delta_scan(act, z, Sz, self.dt_bias, self.a_log, gate, batch, view["state"].state, o, H, G, dk, dv)
        on = rt.buffer("delta_normed", (n, H * dv), rt.dtype)
        ops.wkv_out(o, self.norm, gate, on, H, dv, self.eps)
        stream.add_linear(on, self.w_o)
        return None
