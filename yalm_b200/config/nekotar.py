"""Typed configuration of the Nekotar decoder, read from its ``config.json``.

The design: a token embedding that is RMS-normed; several residual copies per token
("hyper-connections": every sublayer reads one mixture of the copies and writes into all of
them, the output reads their sum); pre-norm layers of three kinds of mixer in any order --
"wkv" (a recurrence with a decay per key channel and a bonus for the current token, fed by
mixtures of each token's input with the previous token's), "latent_attention" (causal attention
whose keys and values are expanded from one cached latent row per token, with a rotated key part
shared by the heads; a layer may read another layer's latent) and "attention" (grouped heads with
biases, rotation of a part of each head, a sliding window that keeps the first tokens visible) --
the last two with an output gate; a GELU feed-forward or none.  Every size and constant is read
from config.json:

    architecture          "Nekotar"
    vocab, width          vocabulary and residual width
    norm.eps              epsilon of every RMS norm
    residual_mult         the factor m on every sublayer's output
    streams               the number of residual copies
    layers[i]             {type: "wkv" | "latent_attention" | "attention", mixer: {...},
                           mlp: null | {kind: "dense", ff}}
      wkv mixer           {heads, dim}   (the decay's inner size is the first dimension of ``w1``)
      latent mixer        {heads, dim, rot_dim, vdim, kv_rank, scale, rot: {base, dims}, kv_from?}
      attention mixer     {heads, kv_heads, dim, vdim, scale, mask: {size, keep_first}, rot: {base, dims}}

Checkpoint tensors: ``embed``, ``embed.norm``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.hc<q>.{in,out,mix}``
(q = 1 the mixer, 2 the feed-forward), ``final.norm``, ``head``; wkv: ``l<i>.mix.mu.{r,k,v,g,w}``,
``l<i>.mix.{r,k,v,g,w1,w2,w0,u,norm,o}``; latent: ``l<i>.mix.{q,dkv,dkv.norm,uk,uv,g,o}`` (no
``dkv*`` with ``kv_from``); attention: ``l<i>.mix.{q,k,v,g,o}`` and ``l<i>.mix.{q,k,v}.b``;
feed-forward: ``l<i>.mlp.{up,down}``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field, replace
from typing import Any, Dict, List, Optional, Tuple

from .llama import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry

NO_POSITION_LIMIT = 1 << 30
DEFAULT_CONTEXT = 1 << 16
DEFAULT_DECAY_RANK = 64          # random-weights mode, when the configuration names none


def _need(d: Dict[str, Any], key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json lacks {where}{key}")
    return d[key]


@dataclass(frozen=True)
class NekotarLayer:
    kind: str                       # "wkv", "latent_attention" or "attention"
    mixer: Dict[str, Any]           # the mixer's own keys, checked
    ff: Optional[int]
    decay_rank: Optional[int] = None


@dataclass(frozen=True)
class NekotarConfig:
    vocab: int
    width: int
    eps: float
    mult: float
    streams: int
    layers: List[NekotarLayer]
    raw: Dict[str, Any] = field(default_factory=dict, compare=False)

    architecture = "Nekotar"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    # ---- reading -------------------------------------------------------------------------
    @staticmethod
    def _rotation(m: Dict[str, Any], where: str, head: int) -> Tuple[float, int]:
        rot = m.get("rot")
        if not rot:
            return 2.0, 0
        base, dims = float(_need(rot, "base", where + "rot.")), int(_need(rot, "dims", where + "rot."))
        if dims % 2 or not 0 <= dims <= head or not base > 1:
            raise ConfigError(f"{where}rot: dims={dims} must be even and at most {head}; base > 1")
        return base, dims

    @classmethod
    def _check_mixer(cls, kind: str, m: Dict[str, Any], where: str, i: int, layers) -> None:
        pos = lambda *keys: [int(_need(m, k, where)) for k in keys]
        if kind == "wkv":
            if min(pos("heads", "dim")) <= 0:
                raise ConfigError(f"{where}: heads and dim must be positive")
        elif kind == "latent_attention":
            heads, dim, rd, vdim, rank = pos("heads", "dim", "rot_dim", "vdim", "kv_rank")
            if min(heads, dim, vdim, rank) <= 0 or rd < 0 or rd % 2:
                raise ConfigError(f"{where}: heads, dim, vdim, kv_rank positive and rot_dim even")
            if not float(_need(m, "scale", where)) > 0:
                raise ConfigError(f"{where}scale must be positive")
            base, dims = cls._rotation(m, where, rd)
            if rd and dims != rd:
                raise ConfigError(f"{where}rot.dims={dims} must equal rot_dim={rd}")
            src = m.get("kv_from")
            if src is not None:
                src = int(src)
                if not 0 <= src < i or layers[src].kind != "latent_attention" \
                        or layers[src].mixer.get("kv_from") is not None:
                    raise ConfigError(f"{where}kv_from={src} must name an earlier latent_attention layer "
                                      f"with a down projection of its own")
                o = layers[src].mixer
                if (int(o["kv_rank"]), int(o["rot_dim"])) != (rank, rd) or cls._rotation(o, where, rd) != (base, dims):
                    raise ConfigError(f"{where}kv_from={src}: kv_rank, rot_dim and rotation must equal that layer's")
        elif kind == "attention":
            heads, kv, dim, vdim = pos("heads", "kv_heads", "dim", "vdim")
            if min(heads, kv, dim, vdim) <= 0 or heads % kv:
                raise ConfigError(f"{where}: heads={heads} must be a positive multiple of kv_heads={kv}")
            if not float(_need(m, "scale", where)) > 0:
                raise ConfigError(f"{where}scale must be positive")
            cls._rotation(m, where, dim)
            mask = m.get("mask") or {}
            if mask and (int(mask.get("size") or 0) <= 0 or int(mask.get("keep_first") or 0) < 0):
                raise ConfigError(f"{where}mask: size must be positive, keep_first not negative")
        else:
            raise ConfigError(f"{where[:-7]}type={kind!r} is not supported ('wkv', 'latent_attention', 'attention')")

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "NekotarConfig":
        layers: List[NekotarLayer] = []
        for i, ld in enumerate(_need(d, "layers", "")):
            where = f"layers[{i}]."
            kind = _need(ld, "type", where)
            mixer = dict(_need(ld, "mixer", where))
            cls._check_mixer(kind, mixer, where + "mixer.", i, layers)
            mlp = ld.get("mlp")
            if mlp and mlp.get("kind", "dense") != "dense":
                raise ConfigError(f"{where}mlp.kind={mlp.get('kind')!r} is not supported (only 'dense')")
            ff = None if not mlp else int(_need(mlp, "ff", where + "mlp."))
            if ff is not None and ff <= 0:
                raise ConfigError(f"{where}mlp.ff must be positive")
            rank = mixer.get("decay_rank")
            layers.append(NekotarLayer(kind, mixer, ff, None if rank is None else int(rank)))
        if not layers:
            raise ConfigError("config.json lists no layers")
        cfg = cls(vocab=int(_need(d, "vocab", "")), width=int(_need(d, "width", "")),
                  eps=float(_need(_need(d, "norm", ""), "eps", "norm.")),
                  mult=float(d.get("residual_mult", 1.0)), streams=int(_need(d, "streams", "")),
                  layers=layers, raw=copy.deepcopy(d))
        if cfg.vocab <= 0 or cfg.width <= 0 or not cfg.eps > 0:
            raise ConfigError("vocab, width and norm.eps must be positive")
        if not 1 <= cfg.streams <= 8:
            raise ConfigError(f"streams={cfg.streams}: 1 to 8 residual copies are supported")
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        d = copy.deepcopy(self.raw)
        for ld, layer in zip(d.get("layers", []), self.layers):
            if layer.kind == "wkv":
                ld["mixer"]["decay_rank"] = layer.decay_rank or DEFAULT_DECAY_RANK
        return d

    def with_tensor_shapes(self, shapes: Dict[str, Tuple[int, ...]]) -> "NekotarConfig":
        """Sizes that only the checkpoint's tensors give: the inner size of a wkv layer's decay
        projection is the first dimension of ``l<i>.mix.w1``."""
        layers = []
        for i, layer in enumerate(self.layers):
            name = f"l{i}.mix.w1"
            if layer.kind == "wkv" and name in shapes and len(shapes[name]) == 2:
                layer = replace(layer, decay_rank=int(shapes[name][0]))
            layers.append(layer)
        return replace(self, layers=layers)

    def ignorable_tensor(self, name: str) -> bool:
        """Tensors of a layer's absent feed-forward sublayer may be in a checkpoint; they are not read."""
        return any(layer.ff is None and (name == f"l{i}.norm2" or name.startswith(f"l{i}.hc2."))
                   for i, layer in enumerate(self.layers))

    # ---- the architecture as a list of parts ---------------------------------------------------
    def _mixer(self, i: int, layer: NekotarLayer) -> PartSpec:
        D, m, p = self.width, layer.mixer, f"l{i}.mix"
        names = lambda *keys: {k: f"{p}.{k}" for k in keys}
        if layer.kind == "wkv":
            return PartSpec("wkv_time_mix",
                            {"hidden_size": D, "num_heads": int(m["heads"]), "key_dim": int(m["dim"]),
                             "value_dim": int(m["dim"]), "decay_rank": layer.decay_rank or DEFAULT_DECAY_RANK,
                             "eps": self.eps},
                            names("mu.r", "mu.k", "mu.v", "mu.g", "mu.w", "r", "k", "v", "g", "w1", "w2", "w0",
                                  "u", "norm", "o"))
        if layer.kind == "latent_attention":
            base, _ = self._rotation(m, "", int(m["rot_dim"]))
            own = m.get("kv_from") is None
            keys = ["q", "uk", "uv", "g", "o"] + (["dkv", "dkv.norm"] if own else [])
            return PartSpec("latent_attention",
                            {"hidden_size": D, "num_heads": int(m["heads"]), "head_dim": int(m["dim"]),
                             "rot_dim": int(m["rot_dim"]), "value_dim": int(m["vdim"]),
                             "kv_rank": int(m["kv_rank"]), "scale": float(m["scale"]), "rot_base": base,
                             "eps": self.eps, "owns_latent": own}, names(*keys))
        base, dims = self._rotation(m, "", int(m["dim"]))
        mask = m.get("mask") or {}
        position = PartSpec("rope_partial", {"head_dim": int(m["dim"]), "dims": dims, "base": base,
                                             "layout": "halves"})
        return PartSpec("gqa_attention",
                        {"hidden_size": D, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]),
                         "head_dim": int(m["dim"]), "value_dim": int(m["vdim"]), "scale": float(m["scale"]),
                         "window": int(mask["size"]) if mask else None,
                         "keep_first": int(mask.get("keep_first") or 0) if mask else None,
                         "bias": True, "element_gate": True, "exact_softmax": True, "position": position},
                        names("q", "k", "v", "g", "o", "q.b", "k.b", "v.b"))

    def to_spec(self) -> ModelSpec:
        D = self.width
        hyper = lambda norm, hc: PartSpec(
            "hyper_rmsnorm", {"size": D, "eps": self.eps, "copies": self.streams, "residual_scale": self.mult},
            {"weight": norm, "in": f"{hc}.in", "out": f"{hc}.out", "mix": f"{hc}.mix"})
        layers, run_order = [], []
        for i, layer in enumerate(self.layers):
            p = f"l{i}"
            parts = {"mixer_norm": hyper(f"{p}.norm1", f"{p}.hc1"), "mixer": self._mixer(i, layer)}
            if layer.ff is not None:
                parts["feed_forward_norm"] = hyper(f"{p}.norm2", f"{p}.hc2")
                parts["feed_forward"] = PartSpec("gelu_mlp", {"hidden_size": D, "intermediate_size": layer.ff},
                                                 {"up": f"{p}.mlp.up", "down": f"{p}.mlp.down"})
            layers.append(LayerSpec("hyper_prenorm", parts))
            src = layer.mixer.get("kv_from") if layer.kind == "latent_attention" else None
            run_order.append(RunEntry(i, reads_cache_of=None if src is None else int(src)))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=D,
            max_positions=NO_POSITION_LIMIT, default_context=DEFAULT_CONTEXT,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "size": D, "norm": {"eps": self.eps}},
                               {"weight": "embed", "norm": "embed.norm"}),
            layers=layers, run_order=run_order,
            final_norm=PartSpec("rmsnorm", {"size": D, "eps": self.eps}, {"weight": "final.norm"}),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "size": D, "tied": False},
                          {"weight": "head"}),
            overlapped_launches=False,
        )
        spec.validate()
        return spec
