"""Typed configuration of the Mufevik architecture: a decoder whose layers carry either two mixers side by side
(softmax attention with weights mixed across heads, and gated linear attention) or a gated delta rule, each followed by
a mixture of experts, around several residual streams per token.

``config.json`` is nested; every size and constant is read from it:

    architecture, vocab, width, streams (absent: one plain residual stream), logit_scale, norm.eps,
    layers[i] = {type: "parallel" | "delta", mixer: {...}, mlp: {...} | null}
    parallel: mixer.left  = {heads, kv_heads, dim, vdim, scale, rot: {dims, base} | absent}
              mixer.right = {heads, dim, vdim, tau}
    delta:    mixer = {heads, kv_heads, dim, vdim, conv}
    mlp = {kind: "moe", router: {experts, top, groups: {count, keep} | absent}, expert: {ff}, shared: {ff} | absent}

Sizes that only tensors give (the rank of the decay's first projection) are read from the checkpoint's shapes.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple, Union

from .base import ConfigError, FieldReader

NAME = "Mufevik"


@dataclass(frozen=True)
class SoftmaxSide:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int                    # 0: no rotation
    rot_base: float

    def to_json(self) -> Dict[str, Any]:
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.rot_dims:
            out["rot"] = {"dims": self.rot_dims, "base": self.rot_base}
        return out


@dataclass(frozen=True)
class LinearSide:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: int                        # rows of the decay's first projection; config key "rank" or the tensor's shape

    def to_json(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "tau": self.tau, "rank": self.rank}


@dataclass(frozen=True)
class ParallelMixer:
    left: SoftmaxSide
    right: LinearSide

    def to_json(self) -> Dict[str, Any]:
        return {"left": self.left.to_json(), "right": self.right.to_json()}


@dataclass(frozen=True)
class DeltaMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    def to_json(self) -> Dict[str, Any]:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}


@dataclass(frozen=True)
class MoeMlp:
    experts: int
    top: int
    group_count: int
    group_keep: int
    expert_ff: int
    shared_ff: int                   # 0: no shared expert

    def to_json(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"kind": "moe", "expert": {"ff": self.expert_ff},
                               "router": {"experts": self.experts, "top": self.top,
                                          "groups": {"count": self.group_count, "keep": self.group_keep}}}
        if self.shared_ff:
            out["shared"] = {"ff": self.shared_ff}
        return out


@dataclass(frozen=True)
class MufevikLayer:
    type: str
    mixer: Union[ParallelMixer, DeltaMixer]
    mlp: Optional[MoeMlp]

    def to_json(self) -> Dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_json(), "mlp": self.mlp.to_json() if self.mlp else None}


@dataclass(frozen=True)
class MufevikConfig:
    vocab: int
    width: int
    norm_eps: float
    streams: int                     # 0: one plain residual stream
    logit_scale: float
    layers: Tuple[MufevikLayer, ...]
    architecture: str = NAME

    MIXER_TYPES = ("parallel", "delta")

    @staticmethod
    def _softmax_side(r: FieldReader) -> SoftmaxSide:
        rot = r.child("rot")
        dims = rot.integer("dims", minimum=0) if rot is not None else 0
        base = rot.number("base", positive=True) if rot is not None else 10000.0
        r.absorb(rot)
        heads, kv = r.integer("heads", minimum=1), r.integer("kv_heads", None, minimum=1)
        dim = r.integer("dim", minimum=1)
        side = SoftmaxSide(heads, kv if kv is not None else heads, dim, r.integer("vdim", dim, minimum=1),
                           r.number("scale", positive=True), dims or 0, base or 10000.0)
        if None not in (side.heads, side.kv_heads, side.dim):
            r.check(side.heads % side.kv_heads == 0, f"'heads' {side.heads} must be a multiple of 'kv_heads' {side.kv_heads}")
            r.check(side.rot_dims % 2 == 0 and side.rot_dims <= side.dim, f"'rot.dims' must be even and at most 'dim' {side.dim}")
        return side

    @classmethod
    def from_dict(cls, data: Dict[str, Any]) -> "MufevikConfig":
        r = FieldReader(data)
        vocab = r.integer("vocab", minimum=1)
        width = r.integer("width", minimum=1)
        streams = r.integer("streams", 0, minimum=0)
        logit_scale = r.number("logit_scale", 1.0)
        norm = r.child("norm")
        eps = norm.number("eps", positive=True) if norm is not None else None
        if norm is None:
            r.check(False, "required key 'norm' is missing")
        r.absorb(norm)
        raw_layers = data.get("layers")
        layers: List[MufevikLayer] = []
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
            elif kind == "parallel":
                left, right = mr.child("left"), mr.child("right")
                if left is None or right is None:
                    mr.check(False, "a parallel mixer needs 'left' and 'right'")
                else:
                    ls = cls._softmax_side(left)
                    rs = LinearSide(right.integer("heads", minimum=1), right.integer("dim", minimum=1),
                                    right.integer("vdim", minimum=1), right.number("tau", positive=True),
                                    right.integer("rank", 0, minimum=0))
                    mr.absorb(left)
                    mr.absorb(right)
                    mixer = ParallelMixer(ls, rs)
            elif kind == "delta":
                heads, kv = mr.integer("heads", minimum=1), mr.integer("kv_heads", None, minimum=1)
                mixer = DeltaMixer(heads, kv if kv is not None else heads, mr.integer("dim", minimum=1),
                                   mr.integer("vdim", minimum=1), mr.integer("conv", minimum=1))
                if None not in (mixer.heads, mixer.kv_heads):
                    mr.check(mixer.heads % mixer.kv_heads == 0, f"'heads' {mixer.heads} must be a multiple of 'kv_heads' {mixer.kv_heads}")
            lr.absorb(mr)
            pr = lr.child("mlp")
            mlp = None
            if pr is not None:
                pr.string("kind", "moe", choices=("moe",))
                router, expert, shared = pr.child("router"), pr.child("expert"), pr.child("shared")
                if router is None or expert is None:
                    pr.check(False, "a mixture of experts needs 'router' and 'expert'")
                else:
                    groups = router.child("groups")
                    count = groups.integer("count", 1, minimum=1) if groups is not None else 1
                    keep = groups.integer("keep", count, minimum=1) if groups is not None else 1
                    router.absorb(groups)
                    mlp = MoeMlp(router.integer("experts", minimum=1), router.integer("top", minimum=1), count, keep,
                                 expert.integer("ff", minimum=1), shared.integer("ff", minimum=1) if shared is not None else 0)
                    if None not in (mlp.experts, mlp.top, count, keep):
                        ok = mlp.experts % count == 0 and keep <= count
                        router.check(ok, f"{mlp.experts} experts must form {count} equal groups of which {keep} are kept")
                        if ok:
                            router.check(mlp.top <= keep * (mlp.experts // count), f"'top' {mlp.top} exceeds the experts of the kept groups")
                pr.absorb(router)
                pr.absorb(expert)
                pr.absorb(shared)
            lr.absorb(pr)
            r.problems.extend(lr.problems)
            if not lr.problems and mixer is not None:
                layers.append(MufevikLayer(kind, mixer, mlp))
        r.finish()
        return cls(vocab, width, float(eps), int(streams), float(logit_scale), tuple(layers))

    @classmethod
    def from_json(cls, path: str) -> "MufevikConfig":
        from .base import read_config_json
        return cls.from_dict(read_config_json(path))

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "norm": {"eps": self.norm_eps}, "logit_scale": self.logit_scale,
                               "layers": [layer.to_json() for layer in self.layers]}
        if self.streams:
            out["streams"] = self.streams
        return out
