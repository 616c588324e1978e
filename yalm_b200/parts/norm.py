"""RMSNorm: o = x * w / sqrt(mean(x^2) + eps), all in 32 bits; the weight
multiplies (no 1 + w), as the reference computes it (infer.cpp:136-146,
infer.cu:525-539).  With ``unit_offset`` the stored weight lies around zero and the norm
multiplies by 1 + w; the sum is formed once, in 32 bits, when the weight is bound."""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from ..weights import TensorNeed
from .base import ResidualStream, register_norm


@register_norm("rmsnorm")
class RMSNorm:
    def __init__(self, params: dict, rt):
        self.rt = rt
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.unit_offset = bool(params.get("unit_offset", False))
        self.weight: Optional[torch.Tensor] = None

    def tensor_needs(self):
        return {"weight": TensorNeed((self.size,), init="around_zero" if self.unit_offset else "ones")}

    def bind(self, tensors) -> None:
        self.weight = self.rt.vector(tensors["weight"])
        if self.unit_offset:
            self.weight = self.weight + 1.0

    def form(self):
        """This norm as ``ops.norm_step`` takes it, for a block that norms a sublayer's output."""
        return (ops.NORM_RMS, self.weight, None, 0.0, self.eps)

    def __call__(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None,
                 n_rows: Optional[int] = None, name: str = "normed") -> torch.Tensor:
        n = stream.x.shape[0] if rows is None else int(n_rows)
        out = self.rt.buffer(name, (n, self.size), self.rt.dtype)
        if stream.due is not None:
            return stream.read_norm(self.form(), out, rows=rows, n_rows=n_rows)
        ops.rmsnorm(stream.x, self.weight, out, self.eps, partials=stream.pending,
                    n_partials=stream.n_pending, rows=rows)
        if rows is None:
            stream.pending, stream.n_pending = None, 0     # folded into x by the kernel
        return out


@register_norm("dynamic_tanh")
class DynamicTanh:
    """A norm that computes no mean and no variance: n(x) = tanh(alpha x) w + b, with a stored scalar
    alpha and a weight and a bias per feature, all in 32 bits.  As a layer's input norm it is called
    like the others; as the norm of a sublayer's output it hands its ``form`` to the stream."""

    def __init__(self, params: dict, rt):
        self.rt = rt
        self.size = int(params["size"])
        self.weight = self.bias = None
        self.alpha = 1.0

    def tensor_needs(self):
        return {"weight": TensorNeed((self.size,), init="ones"), "bias": TensorNeed((self.size,), init="around_zero"),
                "alpha": TensorNeed((), init="ones")}

    def bind(self, tensors) -> None:
        self.weight = self.rt.vector(tensors["weight"])
        self.bias = self.rt.vector(tensors["bias"])
        self.alpha = float(tensors["alpha"].to(torch.float32).reshape(-1)[0])

    def form(self):
        return (ops.NORM_TANH, self.weight, self.bias, self.alpha, 0.0)

    def __call__(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None,
                 n_rows: Optional[int] = None, name: str = "normed") -> torch.Tensor:
        n = stream.x.shape[0] if rows is None else int(n_rows)
        out = self.rt.buffer(name, (n, self.size), self.rt.dtype)
        return stream.read_norm(self.form(), out, rows=rows, n_rows=n_rows)


@register_norm("sum_rmsnorm")
class SumRMSNorm:
    """The norm of a layer that norms AFTER the residual sum: x <- n(a x + y, w), with
    n(v, w) = v / sqrt(mean(v^2) + eps) * w and ``a`` = ``residual_scale``.  y is what the
    sublayer left on the stream: the slices of its last product, or the branches of a mixer
    made of several (each normed with a weight of its own and scaled before the sum).  The new
    x replaces the old in 32 bits; a copy in the compute type is left as ``stream.h`` for the
    next sublayer, which reads x itself."""

    def __init__(self, params: dict, rt):
        self.rt = rt
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.alpha = float(params.get("residual_scale", 1.0))
        self.weight: Optional[torch.Tensor] = None

    def tensor_needs(self):
        return {"weight": TensorNeed((self.size,), init="ones")}

    def bind(self, tensors) -> None:
        self.weight = self.rt.vector(tensors["weight"])

    def apply(self, stream: ResidualStream) -> None:
        if stream.branches:
            branches, beps = stream.branches, stream.branch_eps
        elif stream.n_pending:
            branches, beps = [(stream.pending, stream.n_pending, None, 1.0)], 0.0
        else:
            branches, beps = [], 0.0
        h = None
        if self.rt.dtype != torch.float32:
            h = self.rt.buffer("stream_input", tuple(stream.x.shape), self.rt.dtype)
        ops.sum_norm(stream.x, self.alpha, branches, self.weight, self.eps, h=h, branch_eps=beps)
        stream.pending, stream.n_pending, stream.branches = None, 0, []
        stream.h = h


@register_norm("hyper_rmsnorm")
class HyperRMSNorm:
    """The read and the write of one sublayer in a model with several residual copies X_1 .. X_s
    ("hyper-connections"), around an RMSNorm:

        read:   u = sum_i in[i] X_i;   h = u / sqrt(mean(u^2) + eps) * weight
        write:  X_j <- sum_i mix[i, j] X_i + m out[j] y    (every j from the old copies)

    with y what the sublayer left pending on the stream and m = ``residual_scale``.  The write is
    handed to the stream, which performs it together with the next read (one kernel, one pass)."""

    def __init__(self, params: dict, rt):
        self.rt = rt
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.copies = int(params["copies"])
        self.mult = float(params.get("residual_scale", 1.0))
        if not 1 <= self.copies <= 8:
            raise ValueError(f"hyper_rmsnorm: {self.copies} residual copies (1 to 8)")
        self.weight = self.w_in = self.w_out = self.w_mix = self.ones = None

    def tensor_needs(self):
        s = self.copies
        return {"weight": TensorNeed((self.size,), init="ones"), "in": TensorNeed((s,), init="fraction"),
                "out": TensorNeed((s,), init="ones"), "mix": TensorNeed((s, s), init="identity")}

    def bind(self, tensors) -> None:
        self.weight = self.rt.vector(tensors["weight"])
        self.w_in = self.rt.vector(tensors["in"])
        self.w_out = self.rt.vector(tensors["out"])
        self.w_mix = self.rt.vector(tensors["mix"])
        self.ones = torch.ones(self.copies, dtype=torch.float32, device=self.w_in.device)

    def read(self, stream: ResidualStream, name: str = "normed") -> torch.Tensor:
        if stream.copies is None:
            stream.spread(self.ones)
        out = self.rt.buffer(name, tuple(stream.x.shape), self.rt.dtype)
        return stream.read_copies(self.w_in, self.weight, self.eps, out)

    def write(self, stream: ResidualStream) -> None:
        stream.write_copies(self.w_mix, self.w_out, self.mult)
