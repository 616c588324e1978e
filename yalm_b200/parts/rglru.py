"""A recurrent block around a real-gated linear recurrent unit (the recurrent block of Griffin:
De et al., "Griffin: Mixing Gated Linear Recurrences with Local Attention for Efficient Language
Models"), two branches of ``width`` channels:

    y = gelu(Wy h + by)                                   gelu in its tanh form
    u = conv(Wx h + bx) + bc                              a short causal convolution over time
    r = sigmoid(Ra u + ba),   i = sigmoid(Ri u + bi)      Ra, Ri block-diagonal: ``blocks`` square blocks
    a = exp(-c r softplus(lam)),   S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t      from S = 0, c = ``decay_scale``
    out = Wo (S y)

Two fixed-size cache needs per sequence: S (float32 [width]) and the convolution's last taps - 1
inputs.  The two input projections are one product; the block-diagonal gate products run as one
grouped product whose groups are the blocks (the routed experts' kernel with a fixed plan: block b's
rows are every token's b-th part of u).  Convolution, gates, decay and state are 32-bit.
"""
from __future__ import annotations

import torch

from ..cache import CacheNeed
from ..csrc import ops
from ..weights import TensorNeed
from .base import register_mixer
from .linear import matmul_partials


@register_mixer("rglru_block")
class RglruBlock:
    def __init__(self, params: dict, rt):
        self.rt = rt
        self.D = int(params["hidden_size"])
        self.W = int(params["width"])
        self.blocks = int(params["blocks"])
        self.taps = int(params["conv"])
        self.c = float(params.get("decay_scale", 8.0))
        if min(self.W, self.blocks) <= 0 or self.W % self.blocks or not 2 <= self.taps <= 8:
            raise ValueError(f"rglru_block: {self.W} channels in {self.blocks} equal blocks, convolution of "
                             f"{self.taps} taps (2 to 8)")
        self.bw = self.W // self.blocks
        self.w_yx = self.w_gates = self.w_o = None
        self._plans = {}

    def tensor_needs(self):
        W, D, B, bw = self.W, self.D, self.blocks, self.bw
        zero = lambda *shape: TensorNeed(tuple(shape), init="around_zero")
        return {"y": TensorNeed((W, D)), "y.b": zero(W), "x": TensorNeed((W, D)), "x.b": zero(W),
                "conv": TensorNeed((W, self.taps)), "conv.b": zero(W),
                "ra": TensorNeed((B, bw, bw)), "ra.b": zero(B, bw), "ri": TensorNeed((B, bw, bw)), "ri.b": zero(B, bw),
                "lam": zero(W), "o": TensorNeed((D, W))}

    def bind(self, tensors) -> None:
        rt = self.rt
        yx = [tensors["y"], tensors["x"]]
        gates = [tensors["ra"], tensors["ri"]]
        if any(p.dtype == torch.float32 for p in yx + gates):
            yx, gates = [p.to(torch.float32) for p in yx], [p.to(torch.float32) for p in gates]
        self.w_yx = rt.matrix(torch.cat(yx, 0))
        self.w_gates = rt.matrix(torch.cat(gates, 1))                  # [blocks, 2 bw, bw]: Ra's rows, then Ri's
        self.w_o = rt.matrix(tensors["o"])
        vec = lambda k: rt.vector(tensors[k]).reshape(-1).contiguous()
        self.y_bias, self.x_bias, self.conv_bias = vec("y.b"), vec("x.b"), vec("conv.b")
        self.ra_bias, self.ri_bias, self.lam = vec("ra.b"), vec("ri.b"), vec("lam")
        self.conv_w = rt.vector(tensors["conv"])

    def cache_need(self):
        return {"state": CacheNeed("state", state_shape=(self.W,), state_dtype=torch.float32),
                "conv": CacheNeed("state", state_shape=(self.taps - 1, self.W), state_dtype=torch.float32)}

    def cache_read_bytes(self, contexts, element_size: int) -> int:
        return 2 * len(contexts) * self.taps * self.W * 4

    def flops(self, q_lens, past) -> float:
        return 2.0 * sum(q_lens) * (3 * self.W * self.D + 2 * self.W * self.bw)

    def _plan(self, n: int, tile: int):
        """The grouped product's plan for n tokens: group b owns rows b n .. b n + n - 1, cut into
        tiles of ``tile`` rows.  It depends on n alone and is kept on the device."""
        key = (n, tile)
        if key not in self._plans:
            per = -(-n // tile)
            i32 = dict(dtype=torch.int32, device=self.rt.device)
            first = torch.arange(self.blocks + 1, **i32) * n
            expert = torch.arange(self.blocks, **i32).repeat_interleave(per)
            row0 = (torch.arange(self.blocks, **i32)[:, None] * n + torch.arange(per, **i32)[None, :] * tile).reshape(-1)
            count = torch.tensor([self.blocks * per], **i32)
            if len(self._plans) > 64:
                self._plans.clear()
            self._plans[key] = (first.contiguous(), expert.contiguous(), row0.contiguous(), count, self.blocks * per)
        return self._plans[key]

    def forward(self, h, batch, stream, view, shared: bool = False):
        if shared:
            raise RuntimeError("a recurrent state cannot be read by another run entry")
        rt, W, B, bw = self.rt, self.W, self.blocks, self.bw
        n = batch.n_tokens
        yx, S = matmul_partials(rt, h, self.w_yx, "rglru_yx")
        u = rt.buffer("rglru_u", (n, W), torch.float32)
        u_in = rt.buffer("rglru_u_blocks", (B * n, bw), rt.dtype)        # block-major: the grouped product's rows
        ops.short_conv(yx, S, W, W, self.conv_w, view["conv"].state, batch, out32=u, out16=u_in, block16=bw,
                       in_bias=self.x_bias, out_bias=self.conv_bias)
        gates = rt.buffer("rglru_gates", (B * n, 2 * bw), torch.float32)
        tensor_cores = (rt.gemm != "simt" and u_in.dtype in ops.HALF_TYPES and self.w_gates.dtype == u_in.dtype
                        and bw % 8 == 0)
        if tensor_cores:
            tile = next((t for t in (16, 32, 64) if n <= t), 128)
            ops.gemm_grouped_tc(u_in, self.w_gates, gates, *self._plan(n, tile), tile, rt.status)
        else:
            ops.gemm_grouped(u_in, self.w_gates, gates, *self._plan(n, ops.ROUTED_TILE))
        coef = rt.buffer("rglru_coef", (3, n, W), torch.float32)
        out = rt.buffer("rglru_out", (n, W), rt.dtype)
        ops.rglru(gates, self.ra_bias, self.ri_bias, self.lam, u, yx, S, self.y_bias, coef, batch,
                  view["state"].state, out, W, bw, self.c)
        stream.add_linear(out, self.w_o)
        return None
