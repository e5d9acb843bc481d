"""Typed configuration of the Reravik architecture: a decoder of layers that each carry one of two mixers (a gated
recurrence or a windowed attention over a cached latent), of which a contiguous group may be run several times.

``config.json`` is nested; every size and constant is read from it:

    architecture, vocab, width, embedding.scale, norm.eps,
    layers[i] = {type: "mingru" | "latent_attention", mixer: {...}, mlp: {kind: "dense", ff} | null},
    loop = {start, stop, times}
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple, Union

from .base import ConfigError, FieldReader

NAME = "Reravik"


@dataclass(frozen=True)
class MinGruMixer:
    width: int

    def to_json(self) -> Dict[str, Any]:
        return {"width": self.width}


@dataclass(frozen=True)
class LatentAttentionMixer:
    heads: int
    dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: Optional[int]            # mask.size; None: every earlier token is seen

    def to_json(self) -> Dict[str, Any]:
        out = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "q_rank": self.q_rank, "kv_rank": self.kv_rank,
               "scale": self.scale}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        return out


@dataclass(frozen=True)
class DenseMlp:
    ff: int

    def to_json(self) -> Dict[str, Any]:
        return {"kind": "dense", "ff": self.ff}


@dataclass(frozen=True)
class ReravikLayer:
    type: str
    mixer: Union[MinGruMixer, LatentAttentionMixer]
    mlp: Optional[DenseMlp]

    def to_json(self) -> Dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_json(), "mlp": self.mlp.to_json() if self.mlp else None}


@dataclass(frozen=True)
class ReravikConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[ReravikLayer, ...]
    loop_start: int
    loop_stop: int
    loop_times: int
    architecture: str = NAME

    MIXER_TYPES = ("mingru", "latent_attention")

    @classmethod
    def from_dict(cls, data: Dict[str, Any]) -> "ReravikConfig":
        r = FieldReader(data)
        vocab = r.integer("vocab", minimum=1)
        width = r.integer("width", minimum=2)
        emb = r.child("embedding")
        scale = emb.number("scale", 1.0) if emb is not None else 1.0
        r.absorb(emb)
        norm = r.child("norm")
        eps = norm.number("eps", positive=True) if norm is not None else None
        if norm is None:
            r.check(False, "required key 'norm' is missing")
        r.absorb(norm)
        raw_layers = data.get("layers")
        layers: List[ReravikLayer] = []
        if not isinstance(raw_layers, list) or not raw_layers:
            r.check(False, "'layers' must be a non-empty list")
            raw_layers = []
        for i, raw in enumerate(raw_layers):
            lr = FieldReader(raw, f"config.json:layers[{i}]") if isinstance(raw, dict) else None
            if lr is None:
                r.check(False, f"layers[{i}] must be an object")
                continue
            kind = lr.string("type", choices=cls.MIXER_TYPES)
            mr = lr.child("mixer")
            mixer = None
            if mr is None:
                lr.check(False, "required key 'mixer' is missing")
            elif kind == "mingru":
                mixer = MinGruMixer(mr.integer("width", minimum=1))
            elif kind == "latent_attention":
                mask = mr.child("mask")
                window = mask.integer("size", minimum=1) if mask is not None else None
                mr.absorb(mask)
                mixer = LatentAttentionMixer(mr.integer("heads", minimum=1), mr.integer("dim", minimum=1),
                                             mr.integer("vdim", minimum=1), mr.integer("q_rank", minimum=1),
                                             mr.integer("kv_rank", minimum=1), mr.number("scale", positive=True), window)
            lr.absorb(mr)
            pr = lr.child("mlp")
            mlp = None
            if pr is not None:
                pr.string("kind", choices=("dense",))
                mlp = DenseMlp(pr.integer("ff", minimum=1))
            lr.absorb(pr)
            r.problems.extend(lr.problems)
            if not lr.problems and mixer is not None:
                layers.append(ReravikLayer(kind, mixer, mlp))
        n = len(raw_layers)
        loop = r.child("loop")
        if loop is not None:
            start, stop = loop.integer("start", minimum=0), loop.integer("stop", minimum=0)
            times = loop.integer("times", minimum=1)
            r.absorb(loop)
            if None not in (start, stop, times):
                r.check(start < stop <= n, f"loop: need start < stop <= {n} layers, got start {start}, stop {stop}")
        else:
            start, stop, times = 0, 0, 0            # no repeated group, and no table of pass vectors
        if width is not None:
            r.check(width % 2 == 0, f"'width' must be even (sinusoidal positions come in pairs), got {width}")
        r.finish()
        return cls(vocab, width, float(scale), float(eps), tuple(layers), start, stop, times)

    @classmethod
    def from_json(cls, path: str) -> "ReravikConfig":
        from .base import read_config_json
        return cls.from_dict(read_config_json(path))

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
                               "layers": [layer.to_json() for layer in self.layers]}
        if self.loop_times:
            out["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        return out

    def runs(self) -> List[Tuple[int, Optional[int]]]:
        """The order in which layers run: (layer, number of the pass that begins with this run or None)."""
        n = len(self.layers)
        if not self.loop_times:
            return [(i, None) for i in range(n)]
        out: List[Tuple[int, Optional[int]]] = [(i, None) for i in range(self.loop_start)]
        for t in range(self.loop_times):
            out += [(i, t if i == self.loop_start else None) for i in range(self.loop_start, self.loop_stop)]
        out += [(i, None) for i in range(self.loop_stop, n)]
        return out
