"""SwiGLU feed-forward: x += W2 (silu(W1 h) * (W3 h)), silu(z) = z/(1+exp(-z))
(infer.cpp:356-385, infer.cu:610-634, 936-960).  Gate and up matrices are
kept as one matrix so that one product and its epilogue serve both: when the
width allows it, 16 gate rows are followed by the 16 up rows of the same features
(a tile of the product then holds both halves of each feature); otherwise the up
matrix simply follows the gate matrix.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights import TensorNeed
from .base import register_feed_forward
from .linear import matmul_act, matmul_partials, matmul_silu_mul


@register_feed_forward("swiglu")
class SwiGLU:
    def __init__(self, params: dict, rt):
        self.rt = rt
        self.D = int(params["hidden_size"])
        self.F = int(params["intermediate_size"])
        self.w_gate_up = None
        self.paired = False
        self.w_down = None

    def tensor_needs(self):
        return {"gate": TensorNeed((self.F, self.D)), "up": TensorNeed((self.F, self.D)),
                "down": TensorNeed((self.D, self.F))}

    def bind(self, tensors) -> None:
        parts = [tensors["gate"], tensors["up"]]
        if any(p.dtype == torch.float32 for p in parts):
            parts = [p.to(torch.float32) for p in parts]
        self.paired = self.F % 16 == 0
        if self.paired:
            g, u = (p.reshape(self.F // 16, 16, self.D) for p in parts)
            self.w_gate_up = self.rt.matrix(torch.stack([g, u], 1).reshape(2 * self.F, self.D))
        else:
            self.w_gate_up = self.rt.matrix(torch.cat(parts, 0))
        self.w_down = self.rt.matrix(tensors["down"])

    def flops(self, q_lens, past) -> float:
        return 2.0 * sum(q_lens) * 3 * self.F * self.D

    def forward(self, h, batch, stream) -> None:
        act = self.rt.buffer("ffn_act", (h.shape[0], self.F), self.rt.dtype)
        matmul_silu_mul(self.rt, h, self.w_gate_up, act, self.paired)
        stream.add_linear(act, self.w_down)


@register_feed_forward("gelu_mlp")
class GeluMLP:
    """A feed-forward without a gate: x += Wdown gelu(Wup h), gelu in its tanh form,
    0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))."""

    def __init__(self, params: dict, rt):
        self.rt = rt
        self.D = int(params["hidden_size"])
        self.F = int(params["intermediate_size"])
        self.w_up = self.w_down = None

    def tensor_needs(self):
        return {"up": TensorNeed((self.F, self.D)), "down": TensorNeed((self.D, self.F))}

    def bind(self, tensors) -> None:
        self.w_up = self.rt.matrix(tensors["up"])
        self.w_down = self.rt.matrix(tensors["down"])

    def flops(self, q_lens, past) -> float:
        return 2.0 * sum(q_lens) * 2 * self.F * self.D

    def forward(self, h, batch, stream) -> None:
        act = self.rt.buffer("ffn_act", (h.shape[0], self.F), self.rt.dtype)
        matmul_act(self.rt, h, self.w_up, act, ops.GELU_TANH, "ffn_up")
        stream.add_linear(act, self.w_down)


class ClampedGLU:
    """One gated feed-forward with clamps, y = down(g' sigmoid(slope g') (u' + shift)) with
    g' = min(gate h, limit) and u' = clamp(up h, -limit, limit): the shared expert of a routed
    feed-forward (and, with its constants, any dense feed-forward of that form).  Gate and up
    rows are one matrix laid out as SwiGLU's, and the activation runs where SwiGLU's does: in
    the gate/up product's epilogue, or, where that product is split over K, in the kernel that
    sums the slices."""

    def __init__(self, params: dict, rt, D: int):
        self.rt = rt
        self.D = D
        self.F = int(params["intermediate_size"])
        self.limit = float(params.get("limit") or 0.0)
        self.slope = float(params.get("slope", 1.0))
        self.shift = float(params.get("shift", 0.0))
        self.w_gate_up = None
        self.paired = False
        self.w_down = None

    def tensor_needs(self, prefix: str = ""):
        return {f"{prefix}gate": TensorNeed((self.F, self.D)), f"{prefix}up": TensorNeed((self.F, self.D)),
                f"{prefix}down": TensorNeed((self.D, self.F))}

    def bind(self, gate, up, down) -> None:
        parts = [gate, up]
        if any(p.dtype == torch.float32 for p in parts):
            parts = [p.to(torch.float32) for p in parts]
        self.paired = self.F % 16 == 0
        if self.paired:
            g, u = (p.reshape(self.F // 16, 16, self.D) for p in parts)
            self.w_gate_up = self.rt.matrix(torch.stack([g, u], 1).reshape(2 * self.F, self.D))
        else:
            self.w_gate_up = self.rt.matrix(torch.cat(parts, 0))
        self.w_down = self.rt.matrix(down)

    def flops(self, n_tokens: int) -> float:
        return 2.0 * n_tokens * 3 * self.F * self.D

    def forward(self, h, stream, name: str) -> None:
        act = self.rt.buffer(name + "_act", (h.shape[0], self.F), self.rt.dtype)
        matmul_silu_mul(self.rt, h, self.w_gate_up, act, self.paired,
                        glu=(self.slope, self.limit, self.shift))
        stream.add_linear(act, self.w_down)


@register_feed_forward("routed_experts")
class RoutedExperts:
    """A mixture of experts: router logits z = Wr h and scores = softmax(z) over all experts
    in 32 bits; the experts form ``groups`` equal groups of neighbours, a group's score is its
    largest expert score, only experts of the ``keep_groups`` best groups are eligible, each
    token uses the ``top`` eligible experts with the largest scores, weighted by those scores
    (divided by their sum with ``renormalise``); x += sum_j w_j expert_j(h) + shared(h).
    Other routing rules are parameters: ``score`` "sigmoid" (each logit's own sigmoid instead of the
    softmax), ``correction`` (a stored offset per expert, added to the scores for the choice only; the
    weights use the scores themselves), ``group_score`` "top2" (a group's score is the sum of its two
    best choice scores), ``norm_eps`` (added to the sum the weights are divided by) and
    ``weight_scale`` (a factor on the weights).

    The step: router product -> ``route_topk`` -> ``route_plan`` (the (token, choice) pairs
    sorted by expert, on the device: nothing comes back to the host, so a decode step with
    experts is captured into a graph like any other) -> the tokens' rows gathered in that order
    -> grouped gate/up product -> clamped activation -> grouped down product -> weighted sum
    into the residual stream by token, in the order of the choices."""

    def __init__(self, params: dict, rt):
        self.rt = rt
        self.D = int(params["hidden_size"])
        self.F = int(params["intermediate_size"])
        self.E = int(params["experts"])
        self.top = int(params["top"])
        self.groups = int(params.get("groups") or 1)
        self.keep = int(params.get("keep_groups") or self.groups)
        self.renormalise = bool(params.get("renormalise", False))
        self.limit = float(params.get("limit") or 0.0)
        self.slope = float(params.get("slope", 1.0))
        self.shift = float(params.get("shift", 0.0))
        if params.get("score", "softmax") not in ("softmax", "sigmoid") \
                or params.get("group_score", "max") not in ("max", "top2"):
            raise ValueError("routed_experts: score is 'softmax' or 'sigmoid', group_score 'max' or 'top2'")
        self.sigmoid = params.get("score", "softmax") == "sigmoid"
        self.group_top2 = params.get("group_score", "max") == "top2"
        self.has_correction = bool(params.get("correction", False))
        self.norm_eps = float(params.get("norm_eps") or 0.0)
        self.weight_scale = float(params.get("weight_scale", 1.0))
        self.correction = None
        if self.E % self.groups or not 0 < self.keep <= self.groups:
            raise ValueError(f"{self.E} experts do not form {self.groups} equal groups "
                             f"of which {self.keep} are kept")
        if not 0 < self.top <= self.keep * (self.E // self.groups):
            raise ValueError(f"top={self.top} exceeds the experts of the kept groups")
        self.shared = ClampedGLU(params["shared"], rt, self.D) if params.get("shared") else None
        self.w_router = None
        self.w_gate_up = None          # [E, 2F, D]: gate rows, then up rows, per expert
        self.w_down = None             # [E, D, F]

    def tensor_needs(self):
        needs = {"router": TensorNeed((self.E, self.D))}
        for j in range(self.E):
            needs[f"gate.{j}"] = TensorNeed((self.F, self.D))
            needs[f"up.{j}"] = TensorNeed((self.F, self.D))
            needs[f"down.{j}"] = TensorNeed((self.D, self.F))
        if self.shared is not None:
            needs.update(self.shared.tensor_needs("shared."))
        if self.has_correction:
            needs["correction"] = TensorNeed((self.E,), init="around_zero")
        return needs

    def bind(self, tensors) -> None:
        self.w_router = self.rt.matrix(tensors["router"])
        if self.has_correction:
            self.correction = self.rt.vector(tensors["correction"])
        names = [f"{k}.{j}" for j in range(self.E) for k in ("gate", "up", "down")]
        wide = any(tensors[n].dtype == torch.float32 for n in names)
        get = lambda n: tensors[n].to(torch.float32) if wide else tensors[n]
        self.w_gate_up = self.rt.matrix(torch.stack(
            [torch.cat([get(f"gate.{j}"), get(f"up.{j}")], 0) for j in range(self.E)], 0))
        self.w_down = self.rt.matrix(torch.stack([get(f"down.{j}") for j in range(self.E)], 0))
        if self.shared is not None:
            self.shared.bind(tensors["shared.gate"], tensors["shared.up"], tensors["shared.down"])

    def step_weight_bytes(self, n_tokens: int, element_size: int) -> int:
        """Weight bytes a step of ``n_tokens`` tokens reads: the router, the shared expert, and the
        experts the tokens reach -- as many as independent, evenly spread choices reach on
        average, E (1 - (1 - top/E)^n)."""
        hit = self.E * (1.0 - (1.0 - self.top / self.E) ** n_tokens)
        n = self.E * self.D + int(hit * 3 * self.F * self.D)
        if self.shared is not None:
            n += 3 * self.shared.F * self.D
        return n * element_size

    def flops(self, q_lens, past) -> float:
        n = sum(q_lens)
        total = 2.0 * n * (self.E * self.D + self.top * 3 * self.F * self.D)
        return total + (self.shared.flops(n) if self.shared is not None else 0.0)

    def forward(self, h, batch, stream) -> None:
        from .linear import matmul_partials
        rt, E, top, D, F = self.rt, self.E, self.top, self.D, self.F
        n = h.shape[0]
        pairs = n * top
        i32 = torch.int32
        z, S = matmul_partials(rt, h, self.w_router, "router_logits")
        choice = rt.buffer("routed_choice", (pairs,), i32)
        weight = rt.buffer("routed_weight", (pairs,), torch.float32)
        counts = rt.zeros("routed_counts", E)
        ops.route_topk(z, S, n, E, self.groups, self.keep, top, self.renormalise, choice, weight, counts,
                       sigmoid=self.sigmoid, correction=self.correction, group_top2=self.group_top2,
                       norm_eps=self.norm_eps, weight_scale=self.weight_scale)
        # 16-bit operands that TMA can address: both grouped products on tcgen05, the activation
        # in the first one's epilogue; else the FMA kernel (the 32-bit path among others)
        tensor_cores = (rt.gemm != "simt" and h.dtype in ops.HALF_TYPES and self.w_down.dtype == h.dtype
                        and D % 8 == 0 and F % 8 == 0)
        tile = ops.routed_tile_rows(pairs, E) if tensor_cores else ops.ROUTED_TILE
        max_tiles = ops.routed_max_tiles(pairs, E, tile)
        first_row = rt.buffer("routed_first_row", (E + 1,), i32)
        pair_row = rt.buffer("routed_pair_row", (pairs,), i32)
        row_token = rt.buffer("routed_row_token", (pairs,), i32)
        tile_expert = rt.buffer("routed_tile_expert", (max_tiles,), i32)
        tile_row0 = rt.buffer("routed_tile_row0", (max_tiles,), i32)
        n_tiles = rt.buffer("routed_n_tiles", (1,), i32)
        ops.route_plan(counts, choice, pairs, top, E, first_row, pair_row, row_token, tile_expert,
                       tile_row0, n_tiles, tile_rows=tile)
        plan = (first_row, tile_expert, tile_row0, n_tiles, max_tiles)
        rows = rt.buffer("routed_rows", (pairs, D), h.dtype)
        ops.gather_rows(h, row_token, rows)
        act = rt.buffer("routed_act", (pairs, F), rt.dtype)
        y = rt.buffer("routed_out", (pairs, D), torch.float32)
        if tensor_cores:
            ops.gemm_grouped_tc(rows, self.w_gate_up, act, *plan, tile, rt.status,
                                glu=(self.slope, self.limit, self.shift))
            ops.gemm_grouped_tc(act, self.w_down, y, *plan, tile, rt.status)
        else:
            gu = rt.buffer("routed_gate_up", (pairs, 2 * F), torch.float32)
            ops.gemm_grouped(rows, self.w_gate_up, gu, *plan)
            ops.glu_clamp(gu, act, 1, self.slope, self.limit, self.shift)
            ops.gemm_grouped(act, self.w_down, y, *plan)
        if getattr(stream, "hold", False):
            # the block norms the output before the sum: the weighted sum is formed apart from x
            if self.shared is not None:
                raise RuntimeError("a shared expert beside a held stream is not supported")
            out = rt.buffer("routed_sum", (1, n, D), torch.float32)
            out.zero_()
            ops.routed_combine(out[0], y, pair_row, weight, top)
            stream.pending, stream.n_pending = out, 1
            return
        ops.routed_combine(stream.resolve(), y, pair_row, weight, top)
        if self.shared is not None:
            self.shared.forward(h, stream, "shared_expert")


@register_feed_forward("token_side_input")
class TokenSideInput:
    """A sublayer that feeds the token itself in again: with e the ``dim`` columns from ``first`` of a
    second embedding table's row for the token, y = Wp (gelu(Wg x) * e), gelu in its tanh form.  x is
    what the block hands it (the residual stream itself in a ``prepost_norm`` block's third place);
    the block's output norm takes y from the stream."""

    def __init__(self, params: dict, rt):
        self.rt = rt
        self.D = int(params["hidden_size"])
        self.dim = int(params["dim"])
        self.vocab = int(params["vocab_size"])
        self.table_width = int(params["table_width"])
        self.first = int(params["first"])
        if not 0 <= self.first <= self.table_width - self.dim:
            raise ValueError(f"token_side_input: columns {self.first} .. {self.first + self.dim} of a table "
                             f"{self.table_width} wide")
        self.table = self.w_gate = self.w_proj = None

    def tensor_needs(self):
        return {"table": TensorNeed((self.vocab, self.table_width)), "gate": TensorNeed((self.dim, self.D)),
                "proj": TensorNeed((self.D, self.dim))}

    def bind(self, tensors) -> None:
        self.table = self.rt.matrix(tensors["table"], share=True)
        self.w_gate = self.rt.matrix(tensors["gate"])
        self.w_proj = self.rt.matrix(tensors["proj"])

    def flops(self, q_lens, past) -> float:
        return 2.0 * sum(q_lens) * 2 * self.dim * self.D

    def forward(self, h, batch, stream) -> None:
        rt = self.rt
        z, S = matmul_partials(rt, h, self.w_gate, "side_gate")
        g = rt.buffer("side_gated", (h.shape[0], self.dim), rt.dtype)
        ops.gated_rows(z, S, batch.tokens, self.table, self.first, g)
        stream.add_linear(g, self.w_proj)
