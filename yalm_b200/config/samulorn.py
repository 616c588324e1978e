"""Typed configuration of the Samulorn decoder, read from its ``config.json``.

The design: a scaled token embedding; layers whose sublayers are normed before AND after
(x <- x + n1b(mixer(n1(x))), x <- x + n2b(ff(n2(x)))) by a norm without statistics, tanh(alpha x) w + b;
after the feed-forward every layer feeds the token in again through a small gated projection of a
second embedding table (an RMS norm on its output); two kinds of mixer in any order --
"channel_delta" (the gated delta rule with a decay per key channel, short convolutions on q, k, v)
and "parallel" (grouped-query attention with biases, short convolutions, rotation of neighbouring
pairs with wavelength-band scaling and a weightless norm per head after it, beside a real-gated
linear recurrent unit; the two are added with stored factors) --; a SwiGLU feed-forward, a mixture
of experts (sigmoid scores, a choice offset per expert, groups scored by their two best) or none; a
run of layers may repeat with the same weights.  The head is the embedding table.  Every size and
constant is read from config.json:

    architecture          "Samulorn"
    vocab, width          vocabulary and residual width
    embedding.scale       factor on the looked-up row
    norm.eps              epsilon of the RMS norms (per-head norms, the token input's norm)
    token_side.dim        columns of the second table per layer (absent: no token input)
    loop                  {start, stop, times}: layers start .. stop-1 run `times` times in a row
    layers[i]             {type: "channel_delta" | "parallel", mixer: {...}, mlp: null | {...}}
      channel_delta       {heads, kv_heads, dim, vdim, conv}
      parallel            {left: {heads, kv_heads, dim, vdim, conv, scale, rot: {base, dims, scaling:
                           {factor, low, high, original}}}, right: {width, blocks, conv}, left_scale, right_scale}
      mlp                 {kind: "dense", ff} | {kind: "moe", expert: {ff}, router: {experts, top, scale,
                           groups: {count, keep}}}

Checkpoint tensors: ``embed``, ``side.embed``, ``final.norm{,.b,.alpha}``; per layer ``l<i>.norm{1,1b,2,2b}``
with ``.b`` and ``.alpha``; ``l<i>.side.{gate,proj,norm}``; channel_delta: ``l<i>.mix.{q,k,v}`` and their
``.conv``, ``l<i>.mix.{b,A_log,a1,a2,dt_bias,g1,g2,norm,o}`` (the inner sizes of the two low-rank
projections are the first dimensions of ``a1`` and ``g1``); parallel: ``l<i>.mix.left.{q,k,v}`` with ``.b``
and ``.conv``, ``l<i>.mix.left.o``, ``l<i>.mix.right.{y,y.b,x,x.b,conv,conv.b,ra,ra.b,ri,ri.b,lam,o}``;
feed-forward: ``l<i>.mlp.{gate,up,down}`` or ``l<i>.mlp.{router,correction}`` and ``l<i>.mlp.e<j>.{gate,up,down}``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field, replace
from typing import Any, Dict, List, Optional, Tuple

from .llama import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry

NO_POSITION_LIMIT = 1 << 30
DEFAULT_CONTEXT = 1 << 16
DEFAULT_RANK = 32                # random-weights mode, when neither the configuration nor a tensor names one
RGLRU_DECAY_SCALE = 8.0          # the design's own: log a = -8 r softplus(lam)
ROUTER_SUM_EPS = 1e-20           # the design's own: added to the sum the expert weights are divided by


def _need(d: Dict[str, Any], key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json lacks {where}{key}")
    return d[key]


@dataclass(frozen=True)
class SamulornLayer:
    kind: str                        # "channel_delta" or "parallel"
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]
    decay_rank: Optional[int] = None
    gate_rank: Optional[int] = None


@dataclass(frozen=True)
class SamulornConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    side_dim: int
    layers: List[SamulornLayer]
    loop: Optional[Tuple[int, int, int]]
    raw: Dict[str, Any] = field(default_factory=dict, compare=False)

    architecture = "Samulorn"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    # ---- reading -------------------------------------------------------------------------
    @staticmethod
    def _check_heads(m: Dict[str, Any], where: str) -> None:
        heads, kv, dim, vdim = (int(_need(m, k, where)) for k in ("heads", "kv_heads", "dim", "vdim"))
        if min(heads, kv, dim, vdim) <= 0 or heads % kv:
            raise ConfigError(f"{where}: heads={heads} must be a positive multiple of kv_heads={kv}; dim, vdim positive")
        if not 2 <= int(_need(m, "conv", where)) <= 8:
            raise ConfigError(f"{where}conv={m['conv']}: convolutions of 2 to 8 taps are supported")

    @classmethod
    def _check_layer(cls, kind: str, m: Dict[str, Any], mlp, where: str) -> None:
        if kind == "channel_delta":
            cls._check_heads(m, where + "mixer.")
            if int(m["dim"]) > 256:
                raise ConfigError(f"{where}mixer.dim={m['dim']}: key sizes up to 256 are supported")
        elif kind == "parallel":
            left, right = _need(m, "left", where + "mixer."), _need(m, "right", where + "mixer.")
            cls._check_heads(left, where + "mixer.left.")
            if not float(_need(left, "scale", where + "mixer.left.")) > 0:
                raise ConfigError(f"{where}mixer.left.scale must be positive")
            rot = left.get("rot")
            if rot:
                dims, base = int(_need(rot, "dims", where + "mixer.left.rot.")), float(_need(rot, "base", where + "mixer.left.rot."))
                if dims % 2 or not 0 <= dims <= int(left["dim"]) or not base > 1:
                    raise ConfigError(f"{where}mixer.left.rot: dims={dims} must be even and at most {left['dim']}; base > 1")
                sc = rot.get("scaling")
                if sc:
                    for k in ("factor", "low", "high", "original"):
                        _need(sc, k, where + "mixer.left.rot.scaling.")
                    if float(sc["high"]) == float(sc["low"]):
                        raise ConfigError(f"{where}mixer.left.rot.scaling: low and high must differ")
            width, blocks = int(_need(right, "width", where + "mixer.right.")), int(_need(right, "blocks", where + "mixer.right."))
            if width <= 0 or blocks <= 0 or width % blocks or not 2 <= int(_need(right, "conv", where + "mixer.right.")) <= 8:
                raise ConfigError(f"{where}mixer.right: width={width} in blocks={blocks} equal parts, conv of 2 to 8 taps")
            for k in ("left_scale", "right_scale"):
                float(_need(m, k, where + "mixer."))
        else:
            raise ConfigError(f"{where}type={kind!r} is not supported ('channel_delta', 'parallel')")
        if mlp:
            mk = mlp.get("kind", "dense")
            if mk == "dense":
                if int(_need(mlp, "ff", where + "mlp.")) <= 0:
                    raise ConfigError(f"{where}mlp.ff must be positive")
            elif mk == "moe":
                r = _need(mlp, "router", where + "mlp.")
                E, top = int(_need(r, "experts", where + "mlp.router.")), int(_need(r, "top", where + "mlp.router."))
                g = r.get("groups") or {"count": 1, "keep": 1}
                count, keep = int(g["count"]), int(g["keep"])
                if E <= 0 or count <= 0 or E % count or not 0 < keep <= count or not 0 < top <= keep * (E // count):
                    raise ConfigError(f"{where}mlp.router: experts={E} in {count} groups of which {keep} are kept; top={top}")
                if int(_need(_need(mlp, "expert", where + "mlp."), "ff", where + "mlp.expert.")) <= 0:
                    raise ConfigError(f"{where}mlp.expert.ff must be positive")
            else:
                raise ConfigError(f"{where}mlp.kind={mk!r} is not supported ('dense', 'moe')")

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "SamulornConfig":
        layers: List[SamulornLayer] = []
        for i, ld in enumerate(_need(d, "layers", "")):
            where = f"layers[{i}]."
            kind = _need(ld, "type", where)
            mixer = copy.deepcopy(_need(ld, "mixer", where))
            mlp = copy.deepcopy(ld.get("mlp")) or None
            cls._check_layer(kind, mixer, mlp, where)
            rank = lambda k: None if mixer.get(k) is None else int(mixer[k])
            layers.append(SamulornLayer(kind, mixer, mlp, rank("decay_rank"), rank("gate_rank")))
        if not layers:
            raise ConfigError("config.json lists no layers")
        loop = d.get("loop") or None
        if loop:
            a, b, times = int(_need(loop, "start", "loop.")), int(_need(loop, "stop", "loop.")), int(loop.get("times", 1))
            if not 0 <= a <= b <= len(layers) or times < 1:
                raise ConfigError(f"loop: start={a}, stop={b} must lie within the {len(layers)} layers; times >= 1")
            loop = (a, b, times)
        side = d.get("token_side") or None
        cfg = cls(vocab=int(_need(d, "vocab", "")), width=int(_need(d, "width", "")),
                  eps=float(_need(_need(d, "norm", ""), "eps", "norm.")),
                  embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)),
                  side_dim=int(side["dim"]) if side else 0, layers=layers, loop=loop, raw=copy.deepcopy(d))
        if cfg.vocab <= 0 or cfg.width <= 0 or not cfg.eps > 0 or cfg.side_dim < 0:
            raise ConfigError("vocab, width and norm.eps must be positive")
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        d = copy.deepcopy(self.raw)
        for ld, layer in zip(d.get("layers", []), self.layers):
            if layer.kind == "channel_delta":
                ld["mixer"]["decay_rank"] = layer.decay_rank or DEFAULT_RANK
                ld["mixer"]["gate_rank"] = layer.gate_rank or DEFAULT_RANK
        return d

    def with_tensor_shapes(self, shapes: Dict[str, Tuple[int, ...]]) -> "SamulornConfig":
        """Sizes that only the checkpoint's tensors give: the inner sizes of a channel_delta layer's
        two low-rank projections are the first dimensions of ``l<i>.mix.a1`` and ``l<i>.mix.g1``."""
        layers = []
        for i, layer in enumerate(self.layers):
            if layer.kind == "channel_delta":
                for key, attr in (("a1", "decay_rank"), ("g1", "gate_rank")):
                    name = f"l{i}.mix.{key}"
                    if name in shapes and len(shapes[name]) == 2:
                        layer = replace(layer, **{attr: int(shapes[name][0])})
            layers.append(layer)
        return replace(self, layers=layers)

    def ignorable_tensor(self, name: str) -> bool:
        """The norms of a layer's absent feed-forward may be in a checkpoint; they are not read."""
        return any(layer.mlp is None and name.startswith((f"l{i}.norm2.", f"l{i}.norm2b.")) or
                   layer.mlp is None and name in (f"l{i}.norm2", f"l{i}.norm2b")
                   for i, layer in enumerate(self.layers))

    def run_layers(self) -> List[int]:
        n = len(self.layers)
        if not self.loop:
            return list(range(n))
        a, b, times = self.loop
        return list(range(a)) + list(range(a, b)) * times + list(range(b, n))

    # ---- the architecture as a list of parts ---------------------------------------------------
    def _tanh_norm(self, name: str) -> PartSpec:
        return PartSpec("dynamic_tanh", {"size": self.width},
                        {"weight": name, "bias": name + ".b", "alpha": name + ".alpha"})

    def _mixer(self, i: int, layer: SamulornLayer) -> PartSpec:
        D, m, p = self.width, layer.mixer, f"l{i}.mix"
        if layer.kind == "channel_delta":
            keys = ("q", "k", "v", "q.conv", "k.conv", "v.conv", "b", "A_log", "a1", "a2", "dt_bias", "g1", "g2",
                    "norm", "o")
            return PartSpec("gated_delta_rule",
                            {"hidden_size": D, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]),
                             "key_dim": int(m["dim"]), "value_dim": int(m["vdim"]), "conv": int(m["conv"]),
                             "decay_rank": layer.decay_rank or DEFAULT_RANK,
                             "gate_rank": layer.gate_rank or DEFAULT_RANK, "eps": self.eps},
                            {k: f"{p}.{k}" for k in keys})
        left, right = m["left"], m["right"]
        rot = left.get("rot") or {}
        sc = rot.get("scaling") or None
        scaling = None if not sc else {
            "kind": "llama3", "factor": float(sc["factor"]), "low_freq_factor": float(sc["low"]),
            "high_freq_factor": float(sc["high"]), "original_max_position_embeddings": float(sc["original"])}
        position = PartSpec("rope_partial", {"head_dim": int(left["dim"]), "dims": int(rot.get("dims", 0)),
                                             "base": float(rot.get("base", 2.0)), "layout": "neighbours",
                                             "scaling": scaling})
        attention = PartSpec("gqa_attention",
                             {"hidden_size": D, "num_heads": int(left["heads"]), "num_kv_heads": int(left["kv_heads"]),
                              "head_dim": int(left["dim"]), "value_dim": int(left["vdim"]),
                              "scale": float(left["scale"]), "bias": True, "conv": int(left["conv"]),
                              "head_norm": {"eps": self.eps}, "exact_softmax": True, "position": position})
        recurrent = PartSpec("rglru_block", {"hidden_size": D, "width": int(right["width"]),
                                             "blocks": int(right["blocks"]), "conv": int(right["conv"]),
                                             "decay_scale": RGLRU_DECAY_SCALE})
        tensors = {f"left.{k}": f"{p}.left.{k}" for k in ("q", "k", "v", "o", "q.b", "k.b", "v.b", "q.conv",
                                                          "k.conv", "v.conv")}
        tensors.update({f"right.{k}": f"{p}.right.{k}" for k in ("y", "y.b", "x", "x.b", "conv", "conv.b", "ra",
                                                                 "ra.b", "ri", "ri.b", "lam", "o")})
        return PartSpec("parallel_branches",
                        {"hidden_size": D, "eps": self.eps, "branch_norm": False,
                         "scales": [float(m["left_scale"]), float(m["right_scale"])],
                         "branches": [("left", attention), ("right", recurrent)]}, tensors)

    def _feed_forward(self, i: int, mlp: Dict[str, Any]) -> PartSpec:
        D, p = self.width, f"l{i}.mlp"
        if mlp.get("kind", "dense") == "dense":
            return PartSpec("swiglu", {"hidden_size": D, "intermediate_size": int(mlp["ff"])},
                            {"gate": f"{p}.gate", "up": f"{p}.up", "down": f"{p}.down"})
        r = mlp["router"]
        g = r.get("groups") or {"count": 1, "keep": 1}
        E = int(r["experts"])
        tensors = {"router": f"{p}.router", "correction": f"{p}.correction"}
        for j in range(E):
            tensors.update({f"gate.{j}": f"{p}.e{j}.gate", f"up.{j}": f"{p}.e{j}.up", f"down.{j}": f"{p}.e{j}.down"})
        return PartSpec("routed_experts",
                        {"hidden_size": D, "intermediate_size": int(mlp["expert"]["ff"]), "experts": E,
                         "top": int(r["top"]), "groups": int(g["count"]), "keep_groups": int(g["keep"]),
                         "renormalise": True, "score": "sigmoid", "correction": True, "group_score": "top2",
                         "norm_eps": ROUTER_SUM_EPS, "weight_scale": float(r.get("scale", 1.0))}, tensors)

    def to_spec(self) -> ModelSpec:
        D = self.width
        layers = []
        for i, layer in enumerate(self.layers):
            p = f"l{i}"
            parts = {"mixer_norm": self._tanh_norm(f"{p}.norm1"), "mixer": self._mixer(i, layer),
                     "mixer_post_norm": self._tanh_norm(f"{p}.norm1b")}
            if layer.mlp:
                parts["feed_forward_norm"] = self._tanh_norm(f"{p}.norm2")
                parts["feed_forward"] = self._feed_forward(i, layer.mlp)
                parts["feed_forward_post_norm"] = self._tanh_norm(f"{p}.norm2b")
            if self.side_dim:
                parts["extra"] = PartSpec(
                    "token_side_input",
                    {"hidden_size": D, "dim": self.side_dim, "vocab_size": self.vocab,
                     "table_width": self.side_dim * len(self.layers), "first": i * self.side_dim},
                    {"table": "side.embed", "gate": f"{p}.side.gate", "proj": f"{p}.side.proj"})
                parts["extra_post_norm"] = PartSpec("rmsnorm", {"size": D, "eps": self.eps},
                                                    {"weight": f"{p}.side.norm"})
            layers.append(LayerSpec("prepost_norm", parts))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=D,
            max_positions=NO_POSITION_LIMIT, default_context=DEFAULT_CONTEXT,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "size": D, "scale": self.embedding_scale},
                               {"weight": "embed"}),
            layers=layers, run_order=[RunEntry(i) for i in self.run_layers()],
            final_norm=self._tanh_norm("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "size": D, "tied": True}, {"weight": "embed"}),
            overlapped_launches=False,
        )
        spec.validate()
        return spec
