"""Grouped-query causal attention with an optional sliding window or chunked mask.

q = Wq h, k = Wk h, v = Wv h (one product over the stacked matrix); position
encoding on q and k; k, v into the cache; softmax((q.k)/sqrt(hd)) v over the
visible keys with head h reading kv head h // (H/G); x += Wo o.  The formulas
are the reference's (infer.cpp:278-338, infer.cu:730-920); the window
(keys p-W+1..p) is the checkpoint's ``sliding_window``, which the reference
does not read.

Options beyond that, each a parameter (all off for the Llama / Mistral decoder):

* ``scale``: the factor on q.k in place of 1/sqrt(hd);
* ``chunk``: a query at position p sees the keys j <= p of its own chunk,
  p // chunk == j // chunk, chunks counted from position 0 of the sequence.  Keys of
  earlier chunks are never read again, so the cache keeps a ring of ``chunk`` rows per
  sequence (position p at row p % chunk), as it keeps ``window`` rows under a window;
* ``value_dim``: a value size that differs from the query/key size.  The kernels take one
  head size, so the smaller of the two is padded with zero rows of the weights (zero
  columns of Wo): scores and outputs are unchanged, and nothing is padded when they agree.
  Only an encoding without rotation allows it (rotation pairs depend on the head size);
* ``head_gate``: head h's output is multiplied by sigmoid(Wg h)_h, Wg [H, width], before Wo;
* ``element_gate``: the concatenated heads are multiplied feature by feature by sigmoid(Wg h),
  Wg [H * value size, width], before Wo;
* ``qk_norm`` = {"eps": e}: q and k are each normed over the WHOLE projection (all heads of a
  token at once) with weights ``q.norm`` / ``k.norm`` of that size, before rotation (needs the
  ``rope_partial`` position encoding, whose kernel does both);
* ``head_temp``: head h's scores are multiplied by ``temp``[h]; the factor is folded into head
  h's part of the ``q.norm`` weight in 32 bits when the weights are bound;
* ``values_from_keys``: there is no v projection; a position's value is its key as projected,
  before norm and rotation;
* ``pool`` = P (with a window W): beside the last W positions a query sees one (mean key, mean
  value) for every block of P positions that lies wholly before its window (block b if
  b P + P - 1 <= pos - W), in the same softmax.  The means are formed from the rows as the
  cache holds them when a block completes, and live in a second cache with one row per block;
  the ring of the window keeps max(W, P) rows so that a completing block's rows are still there;
* ``bias``: q, k and v have biases (``q.b``, ``k.b``, ``v.b``), added where the product's slices are summed;
* ``keep_first`` = F (with a window W): a query also sees the positions below F, at their own
  positions (for rotation and distance), however far back they lie.  The cache then keeps every
  position instead of a ring of W rows;
* ``conv`` = taps: a short causal convolution over time on every channel of q, k and v
  (``q.conv``, ``k.conv``, ``v.conv`` [channels, taps], the last column the current token's), directly
  after the projection and its bias, before norm and rotation; the last taps - 1 projected rows of
  a sequence are a fixed-size cache need beside its keys and values;
* ``head_norm`` = {"eps": e}: after the rotation every head of q and k is divided by its own root mean
  square (a norm without a weight; needs the ``rope_partial`` encoding);
* ``exact_softmax``: scores, softmax weights and the weighted sum of values in 32-bit arithmetic
  (the FMA attention kernels on the 16-bit cache) instead of the tensor-core kernels, whose
  weights are rounded to 16 bits.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..cache import CacheNeed
from ..csrc import ops
from ..weights import TensorNeed
from .base import POSITIONS, make_part, register_mixer
from . import decode_plan, linear
from .linear import matmul_partials


def exact_attention(rt, q, kv_step, k_cache, v_cache, batch, slot_pos, o, H, G, hd, capacity, window, pages,
                    scale, chunk=None, pooled=None, pool=None, keep_first=None) -> None:
    """Attention with 32-bit scores, softmax weights and weighted sum: a prompt (or a portion of
    one) on the tensor-core kernel that carries every weight as three 16-bit terms, where that
    kernel takes the shape; else the FMA kernel, a decode step's few queries split over their keys
    so that the grid fills the device."""
    n = batch.n_tokens
    if (not batch.is_decode and rt.attention != "simt"
            and ops.exact_attention_usable(rt.dtype, hd, chunk)):
        ops.attention_exact_prefill(q, kv_step, k_cache, v_cache, batch, slot_pos, o, H, G, hd, capacity,
                                    window, pages=pages, scale=scale, pooled=pooled, keep_first=keep_first)
        return
    bound = max(1, batch.ctx_bound)
    span = window or chunk
    visible = min(bound, span) if span else bound
    if pool:
        visible += bound // pool
    if keep_first:
        visible = min(bound, visible + keep_first)
    nsplit = 1
    if batch.is_decode:
        blocks = n * G * -(-(H // G) // 4)
        nsplit = max(1, min(-(-visible // 64), 2 * rt.sm_count // max(1, blocks), 64))
    part_o = rt.buffer("attn_part_o", (n, H, nsplit, hd), torch.float32)
    part_ml = rt.buffer("attn_part_ml", (n, H, nsplit, 2), torch.float32)
    ops.attention(q, kv_step, k_cache, v_cache, batch, slot_pos, o, H, G, hd, capacity, window, nsplit,
                  part_o, part_ml, pages=pages, pooled=pooled, chunk=chunk, scale=scale, keep_first=keep_first)


@register_mixer("gqa_attention")
class GQAAttention:
    def __init__(self, params: dict, rt):
        self.rt = rt
        self.D = int(params["hidden_size"])
        self.H = int(params["num_heads"])
        self.G = int(params["num_kv_heads"])
        self.hd_k = int(params["head_dim"])
        self.hd_v = int(params.get("value_dim") or self.hd_k)
        self.window: Optional[int] = params.get("window") or None
        self.chunk: Optional[int] = params.get("chunk") or None
        self.scale: Optional[float] = params.get("scale") or None
        self.head_gate = bool(params.get("head_gate", False))
        self.element_gate = bool(params.get("element_gate", False))
        self.qk_norm = params.get("qk_norm") or None
        self.head_temp = bool(params.get("head_temp", False))
        self.values_from_keys = bool(params.get("values_from_keys", False))
        self.pool: Optional[int] = params.get("pool") or None
        self.exact = bool(params.get("exact_softmax", False))
        self.bias = bool(params.get("bias", False))
        self.keep_first: Optional[int] = params.get("keep_first") or None
        self.conv: Optional[int] = int(params["conv"]) if params.get("conv") else None
        self.head_norm = params.get("head_norm") or None
        if (self.conv or self.head_norm) and params["position"].kind != "rope_partial":
            raise ValueError("a convolution after the projection and a norm per head after the rotation "
                             "need the rope_partial encoding")
        if self.conv is not None and not 2 <= self.conv <= 8:
            raise ValueError(f"a convolution of {self.conv} taps (2 to 8)")
        if self.head_norm and params.get("qk_norm"):
            raise ValueError("a norm per head and whole-projection norms exclude each other")
        if self.keep_first and not self.window:
            raise ValueError("kept first positions stay visible beside a sliding window: the mixer needs one")
        if self.keep_first and self.pool:
            raise ValueError("kept first positions and pooled blocks exclude each other")
        if self.bias and params["position"].kind != "rope_partial":
            raise ValueError("biases of q, k and v are added by the rope_partial encoding's kernel")
        if self.head_gate and self.element_gate:
            raise ValueError("a gate per head and a gate per feature exclude each other")
        if self.pool and not self.window:
            raise ValueError("pooled blocks lie before a sliding window: the mixer needs one")
        if self.values_from_keys and self.hd_v != self.hd_k:
            raise ValueError(f"values that are the keys have the keys' size {self.hd_k}, not {self.hd_v}")
        if (self.qk_norm or self.values_from_keys) and params["position"].kind != "rope_partial":
            raise ValueError("whole-projection norms and values from keys need the rope_partial encoding")
        if self.head_temp and not self.qk_norm:
            raise ValueError("a factor per head is folded into the q norm's weight: the mixer needs qk_norm")
        if self.window and self.chunk:
            raise ValueError("a sliding window and a chunked mask exclude each other")
        if self.H % self.G:
            raise ValueError(f"{self.H} heads do not divide into {self.G} kv heads")
        position = params["position"]
        # the one head size the kernels run with
        self.hd = max(self.hd_k, self.hd_v)
        if self.hd_k != self.hd_v or self.hd % 8:
            if position.kind not in ("none", "rope_partial"):
                raise ValueError(f"head sizes {self.hd_k} (keys) and {self.hd_v} (values) need padding "
                                 f"to one multiple of 8, which a rotating position encoding rules out")
            self.hd = -(-self.hd // 16) * 16
            position = type(position)(position.kind, {**position.params, "head_dim": self.hd},
                                      position.tensors)
        if not 0 < self.hd <= 256:
            raise ValueError(f"head size {self.hd} is not supported by the attention kernel "
                             f"(up to 256)")
        self.span = self.window or self.chunk          # the most keys a query sees, if bounded
        if self.keep_first:
            self.span = None                           # no ring: see ``cache_need``
        if position.kind == "rope_partial" and int(position.params.get("head_dim", self.hd)) != self.hd:
            position = type(position)(position.kind, {**position.params, "head_dim": self.hd},
                                      position.tensors)
        self.position = make_part(POSITIONS, position, rt)
        self.q_norm = self.k_norm = None
        self._store_extras = {}
        self.w_qkv = None
        self.w_o = None
        self.w_g = None

    def tensor_needs(self):
        needs = {"q": TensorNeed((self.H * self.hd_k, self.D)),
                 "k": TensorNeed((self.G * self.hd_k, self.D)),
                 "v": TensorNeed((self.G * self.hd_v, self.D)),
                 "o": TensorNeed((self.D, self.H * self.hd_v))}
        if self.values_from_keys:
            del needs["v"]
        if self.head_gate:
            needs["g"] = TensorNeed((self.H, self.D))
        if self.element_gate:
            needs["g"] = TensorNeed((self.H * self.hd_v, self.D))
        if self.qk_norm:
            needs["q.norm"] = TensorNeed((self.H * self.hd_k,), init="ones")
            needs["k.norm"] = TensorNeed((self.G * self.hd_k,), init="ones")
        if self.head_temp:
            needs["temp"] = TensorNeed((self.H,), init="ones")
        if self.bias:
            needs["q.b"] = TensorNeed((self.H * self.hd_k,), init="around_zero")
            needs["k.b"] = TensorNeed((self.G * self.hd_k,), init="around_zero")
            if not self.values_from_keys:
                needs["v.b"] = TensorNeed((self.G * self.hd_v,), init="around_zero")
        if self.conv:
            needs["q.conv"] = TensorNeed((self.H * self.hd_k, self.conv))
            needs["k.conv"] = TensorNeed((self.G * self.hd_k, self.conv))
            if not self.values_from_keys:
                needs["v.conv"] = TensorNeed((self.G * self.hd_v, self.conv))
        return needs

    def _pad_vector(self, w: torch.Tensor, heads: int, size: int) -> torch.Tensor:
        """float32 [heads * size] -> [heads * hd] with zeros after each head's own."""
        w = self.rt.vector(w)
        if size == self.hd:
            return w
        out = torch.zeros((heads, self.hd), dtype=torch.float32, device=w.device)
        out[:, :size] = w.view(heads, size)
        return out.view(-1).contiguous()

    def _pad_heads(self, w: torch.Tensor, heads: int, size: int) -> torch.Tensor:
        """[heads * size, D] -> [heads * hd, D] with zero rows after each head's own."""
        if size == self.hd:
            return w
        out = torch.zeros((heads, self.hd, w.shape[1]), dtype=w.dtype, device=w.device)
        out[:, :size] = w.view(heads, size, w.shape[1])
        return out.view(heads * self.hd, w.shape[1])

    def bind(self, tensors) -> None:
        parts = [self._pad_heads(tensors["q"], self.H, self.hd_k),
                 self._pad_heads(tensors["k"], self.G, self.hd_k)]
        if not self.values_from_keys:
            parts.append(self._pad_heads(tensors["v"], self.G, self.hd_v))
        if any(p.dtype == torch.float32 for p in parts):
            parts = [p.to(torch.float32) for p in parts]
        self.w_qkv = self.rt.matrix(torch.cat(parts, 0))
        w_o = tensors["o"]
        if self.hd_v != self.hd:
            padded = torch.zeros((self.D, self.H, self.hd), dtype=w_o.dtype, device=w_o.device)
            padded[:, :, :self.hd_v] = w_o.view(self.D, self.H, self.hd_v)
            w_o = padded.view(self.D, self.H * self.hd)
        self.w_o = self.rt.matrix(w_o)
        if self.head_gate:
            self.w_g = self.rt.matrix(tensors["g"])
        if self.element_gate:
            self.w_g = self.rt.matrix(self._pad_heads(tensors["g"], self.H, self.hd_v))
        if self.qk_norm:
            self.q_norm = self._pad_vector(tensors["q.norm"], self.H, self.hd_k)
            self.k_norm = self._pad_vector(tensors["k.norm"], self.G, self.hd_k)
            if self.head_temp:
                temp = self.rt.vector(tensors["temp"])
                self.q_norm = (self.q_norm.view(self.H, self.hd) * temp[:, None]).reshape(-1).contiguous()
            self._store_extras["norms"] = (self.q_norm, self.k_norm, self.H * self.hd_k,
                                           self.G * self.hd_k, float(self.qk_norm["eps"]))
        if self.values_from_keys:
            self._store_extras["has_v"] = False
        if self.bias:
            b = [self._pad_vector(tensors["q.b"], self.H, self.hd_k), self._pad_vector(tensors["k.b"], self.G, self.hd_k)]
            if not self.values_from_keys:
                b.append(self._pad_vector(tensors["v.b"], self.G, self.hd_v))
            self._store_extras["bias"] = torch.cat(b).contiguous()
        if self.conv:
            c = [self._pad_heads(self.rt.vector(tensors["q.conv"]), self.H, self.hd_k),
                 self._pad_heads(self.rt.vector(tensors["k.conv"]), self.G, self.hd_k)]
            if not self.values_from_keys:
                c.append(self._pad_heads(self.rt.vector(tensors["v.conv"]), self.G, self.hd_v))
            self.conv_w = torch.cat(c, 0).contiguous()
        if self.head_norm:
            self._store_extras["head_norm"] = (float(self.head_norm["eps"]), self.hd_k)

    def _kv_need(self):
        if self.keep_first:
            # every position stays (the first ones are seen for ever); the mask alone bounds the keys
            return CacheNeed("kv", kv_heads=self.G, head_dim=self.hd, window=None)
        if not self.pool:
            return CacheNeed("kv", kv_heads=self.G, head_dim=self.hd, window=self.span)
        # the ring keeps a completing block's rows; the pooled rows are never dropped
        return {"kv": CacheNeed("kv", kv_heads=self.G, head_dim=self.hd, window=max(self.window, self.pool)),
                "pool": CacheNeed("kv", kv_heads=self.G, head_dim=self.hd, window=None, every=self.pool)}

    def cache_need(self):
        need = self._kv_need()
        if not self.conv:
            return need
        rows = (self.H + (1 if self.values_from_keys else 2) * self.G) * self.hd
        needs = dict(need) if isinstance(need, dict) else {"kv": need}
        needs["conv"] = CacheNeed("state", state_shape=(self.conv - 1, rows), state_dtype=torch.float32)
        return needs

    def decode_chunk(self, batch) -> int:
        """Keys per block of the decode kernel: 64 KiB of keys and values, so
        that three blocks share an SM and hide each other's copy latency."""
        esz = 4 if self.rt.dtype == torch.float32 else 2
        chunk = (64 * 1024) // (2 * self.hd * esz)
        return max(8, min(128, chunk))

    def planned_chunks(self, batch):
        """64-key chunks of every sequence as the decode kernel's plan counts them: at the
        lengths the sequences will have when the longest reaches the step's context bound.
        A captured decode step keeps its plan until then, and a plan made for today's lengths
        goes wrong on the way: sequences of equal length that outgrow their block's run by one
        chunk all split in two, the grid doubles and every query is merged (measured at 7B
        sizes, 16 sequences of 700 keys: 3.46 against 3.10 ms per step)."""
        slack = max(0, max(1, batch.ctx_bound) - (max(batch.past) + 1))
        return [-(-(min(p + 1 + slack, self.span) if self.span else p + 1 + slack) // 64)
                for p in batch.past]

    def decode_chunks_per_block(self, batch, visible: int) -> int:
        """How many 64-key chunks one block of the tensor-core decode kernel walks
        through: the fewest with which all blocks are resident at once (one per
        SM; its four warps take the chunks' halves in turn), but no fewer than
        leave a sequence about six parts, and a whole sequence of up to eight
        chunks (lengths as they are when the longest reaches the step's bound).
        A few sequences then get several blocks each and a merge; with many
        sequences a block takes its whole sequence and nothing is merged.
        (Merging costs about 2 us and 0.3 to 0.4 us per part, a further unit of 32
        keys per warp about 1 us: one or two sequences of 1,000 to 4,000 keys in
        16 parts each, as the first rule alone has it, take 2.5 to 4 % longer per
        step at 7B sizes than in 6; a sequence of 300 keys in 5 parts 1.5 to 2 %
        longer than in one.)"""
        groups = self.G * -(-(self.H // self.G) // 16)
        chunks = self.planned_chunks(batch)
        resident = self.rt.sm_count
        most = max(1, -(-visible // 64))
        if self.rt.decode_attention_chunks:
            return min(most, int(self.rt.decode_attention_chunks))
        cpc = max(1, min(most, -(-groups * sum(chunks) // resident)))
        while cpc < most and groups * sum(-(-c // cpc) for c in chunks) > resident:
            cpc += 1
        longest = max(chunks)
        return max(cpc, most if longest <= 8 else min(most, -(-most // 6)))

    def decode_warps(self, batch, visible: int, cpc: int) -> int:
        """Warps per block of the tensor-core decode kernel: four, unless the blocks take
        whole sequences, outnumber the SMs' block slots, and the estimate of
        ``decode_plan`` says that two blocks of two warps per SM get through the grid
        sooner (few long blocks of equal length; many waves)."""
        if self.rt.decode_attention_warps:
            return int(self.rt.decode_attention_warps)
        if cpc < max(1, -(-visible // 64)):
            return 4
        chunks = tuple(self.planned_chunks(batch))
        groups = self.G * -(-(self.H // self.G) // 16)
        return decode_plan.decode_warps(decode_plan.rounded(chunks), groups, self.hd,
                                        self.rt.sm_count)

    # The decode kernel's grid takes sequences in row order, and long blocks that start
    # last leave the SMs idle at the end: the generation loop orders a batch by this.
    prefers_longest_first = True

    def cache_read_bytes(self, contexts, element_size: int) -> int:
        """Bytes of keys and values one decode step reads for sequences of these lengths."""
        if self.chunk:
            seen = sum((c - 1) % self.chunk + 1 for c in contexts if c > 0)
        else:
            seen = sum(min(c, self.window) if self.window else c for c in contexts)
        if self.pool:
            seen += sum(max(0, c - self.window) // self.pool for c in contexts)
        return seen * 2 * self.G * self.hd * element_size

    def flops(self, q_lens, past) -> float:
        """Multiply-adds times two of a step: the four projections and, for each query,
        scores and value mix over the keys it sees."""
        n = sum(q_lens)
        kv = 1 if self.values_from_keys else 2
        linear = 2.0 * n * ((self.H + kv * self.G) * self.hd * self.D + self.D * self.H * self.hd
                            + (self.H * self.D if self.head_gate else 0)
                            + (self.H * self.hd * self.D if self.element_gate else 0))
        pairs = 0
        for q, p in zip(q_lens, past):
            for pos in range(p, p + q):
                if self.chunk:
                    pairs += pos % self.chunk + 1
                else:
                    pairs += min(pos + 1, self.window) if self.window else pos + 1
                    if self.pool:
                        pairs += max(0, pos - self.window + 1) // self.pool
        return linear + 4.0 * self.H * self.hd * pairs

    def forward(self, h, batch, stream, view, shared: bool = False):
        rt, H, G, hd = self.rt, self.H, self.G, self.hd
        n = batch.n_tokens
        pool_view = conv_view = None
        if isinstance(view, dict):
            pool_view, conv_view, view = view.get("pool"), view.get("conv"), view["kv"]
        extras = self._store_extras
        if self.conv and shared:
            raise RuntimeError("a convolved projection cannot read another run entry's cache")
        q = rt.buffer("q_rot", (n, H * hd), rt.dtype)
        # many tokens: the q/k/v product rotates and stores in its own epilogue
        table = getattr(self.position, "step_table", None)
        fused = (not shared and n > linear.MANY_TOKENS and table is not None and rt.gemm != "simt"
                 and ops.gemm_2sm_rope_usable(h, self.w_qkv, hd))
        if not fused:
            qkv, S = matmul_partials(rt, h, self.w_qkv, "qkv")
        if self.conv:
            # bias, then the convolution over time, in 32 bits; the store kernel goes on from its output
            rows = self.w_qkv.shape[0]
            conv = rt.buffer("qkv_conv", (1, n, rows), torch.float32)
            ops.short_conv(qkv, S, 0, rows, self.conv_w, conv_view.state, batch, out32=conv[0],
                           in_bias=extras.get("bias"))
            qkv, S = conv, 1
            extras = {k: v for k, v in extras.items() if k != "bias"}
        if self.head_gate or self.element_gate:
            gate, gate_S = matmul_partials(rt, h, self.w_g, "head_gate")
        mask = {"chunk": self.chunk, "scale": self.scale}
        dmask = {"mask_chunk": self.chunk, "scale": self.scale}
        tensor_cores = (ops.mma_attention_usable(rt.dtype, hd) and rt.attention != "simt"
                        and not self.exact and not self.pool)
        # one token per sequence on the tensor-core kernel, a small batch: that kernel sums the
        # product's slices, rotates and writes the cache row itself (no rotary kernel, one
        # hand-over less: 2-3 % of a step at batch 1, 0.5 % at 8 to 16; from 32 sequences on the
        # rotary kernel's many small blocks are the faster way, by 1-2 %)
        in_attention = (batch.is_decode and n <= 16 and tensor_cores and not shared and not fused
                        and table is not None and getattr(view, "kv_step", None) is None
                        and getattr(rt, "decode_rope_in_attention", True))
        # a layer whose cache another run entry reads keeps its step keys apart
        kv_step = view.kv_step if getattr(view, "kv_step", None) is not None else \
            rt.buffer("kv_step", (n, 2, G, hd), rt.dtype)
        # Several tokens on top of a ring that is already full: their rows would
        # replace keys that the first of them still has to see, so the ring is
        # written after the attention instead of before it -- and after every later
        # run entry that reads this cache: then the write is handed back to the model.
        late_write = (not shared) and any(
            p > 0 and ql > 1 and p + ql > view.capacity for p, ql in zip(batch.past, batch.q_lens))
        if fused:
            ops.gemm_2sm_rope(h, self.w_qkv, table(batch, view.slot_pos), batch, q, kv_step, view.k,
                              view.v, view.slot_pos,
                              H, G, hd, view.capacity, rt.status, write_cache=not late_write,
                              pages=view.pages)
        elif in_attention:
            pass
        elif shared:
            # this run reads the owner's keys and values: rotate q only
            scratch = rt.buffer("kv_step_unused", (n, 2, G, hd), rt.dtype)
            self.position.rotate_and_store(qkv, S, batch, view, q, scratch, H, G,
                                           write_cache=False, **extras)
        else:
            self.position.rotate_and_store(qkv, S, batch, view, q, kv_step, H, G,
                                           write_cache=not late_write, **extras)
        pooled = None
        if self.pool:
            # the blocks this step completes, before any query of the step looks at them (and
            # before the late ring write, which may replace rows they are made of)
            if not shared and view.capacity >= self.pool - 1:
                ops.pool_blocks(kv_step, view.k, view.v, batch, view.slot_pos, pool_view.k, pool_view.v,
                                G, hd, view.capacity, self.pool, pool_view.capacity, rt.status,
                                pages=view.pages, pool_pages=pool_view.pages)
            pooled = (pool_view.k, pool_view.v, self.pool, pool_view.capacity, pool_view.pages)
        o = rt.buffer("attn_out", (n, H * hd), rt.dtype)
        if self.pool or self.keep_first or (self.exact and not batch.is_decode):
            # 32-bit scores, weights and sums over the window's rows, the pooled rows and the kept
            # first positions
            exact_attention(rt, q, kv_step, view.k, view.v, batch, view.slot_pos, o, H, G, hd, view.capacity,
                            self.window, view.pages, self.scale, chunk=self.chunk, pooled=pooled,
                            pool=self.pool, keep_first=self.keep_first)
        elif batch.is_decode:
            # one query per sequence, every key already in the cache
            bound = max(1, batch.ctx_bound)
            visible = min(bound, self.span) if self.span else bound
            if tensor_cores:
                cpc = self.decode_chunks_per_block(batch, visible)
                warps = 4 if in_attention else self.decode_warps(batch, visible, cpc)
                parts = ops.decode_mma_parts(bound, self.window, cpc, self.chunk)
            else:
                chunk = self.decode_chunk(batch)
                parts = -(-visible // chunk)
            part_o = rt.buffer("attn_part_o", (n, H, parts, hd), torch.float32)
            part_ml = rt.buffer("attn_part_ml", (n, H, parts, 2), torch.float32)
            counters = rt.zeros("attn_counters", n * G * -(-(H // G) // 4))
            if in_attention:
                ops.attention_decode_mma_fused(qkv, S, table(batch, view.slot_pos), view.k, view.v,
                                               batch.seq_slot, view.slot_pos, o, part_o, part_ml,
                                               counters, rt.status, H, G, hd, view.capacity,
                                               self.window, bound, cpc, pages=view.pages, **dmask)
            elif tensor_cores:
                ops.attention_decode_mma(q, view.k, view.v, batch.seq_slot, view.slot_pos, o,
                                         part_o, part_ml, counters, rt.status, H, G, hd,
                                         view.capacity, self.window, bound, cpc, pages=view.pages,
                                         warps=warps, **dmask)
            else:
                ops.attention_decode(q, view.k, view.v, batch.seq_slot, view.slot_pos, o, part_o,
                                     part_ml, counters, rt.status, H, G, hd, view.capacity,
                                     self.window, chunk, bound, pages=view.pages, **dmask)
        elif rt.attention in ("auto", "tcgen05") and not self.exact and ops.tc_attention_usable(
                rt.dtype, hd, batch.past, batch.q_lens, view.capacity):
            # S, P and O in tensor memory, two query tiles per block in ping-pong (41 us
            # against 357 us for the mma.sync kernel per layer at 2,048 tokens of 32 heads
            # of 128).  Whole prompts read this step's own keys; prompts that go on (and do
            # not wrap around their ring in this step) read every key from the cache, which
            # holds this step's rows by now.
            if all(p == 0 for p in batch.past):
                ops.attention_prefill_tc(q, kv_step, batch, o, H, G, hd, self.window, rt.status, **mask)
            else:
                ops.attention_prefill_tc_cache(q, view.k, view.v, batch, view.slot_pos, o, H, G, hd,
                                               view.capacity, self.window, rt.status, pages=view.pages,
                                               **mask)
        elif tensor_cores:
            ops.attention_prefill_mma(q, kv_step, view.k, view.v, batch, view.slot_pos, o, H, G,
                                      hd, view.capacity, self.window, pages=view.pages, **mask)
        else:
            ops.attention(q, kv_step, view.k, view.v, batch, view.slot_pos, o, H, G, hd,
                          view.capacity, self.window, 1, None, None, pages=view.pages, **mask)
        if self.head_gate:
            ops.head_gate(o, gate, gate_S, H, hd)
        elif self.element_gate:
            ops.element_gate(o, gate, gate_S)
        stream.add_linear(o, self.w_o)
        if late_write:
            def write_ring():
                ops.cache_write(kv_step, batch, view.k, view.v, view.slot_pos, G, hd, view.capacity,
                                pages=view.pages)
            if getattr(view, "kv_step", None) is not None:
                return write_ring                  # other run entries still read the old rows
            write_ring()
        return None
