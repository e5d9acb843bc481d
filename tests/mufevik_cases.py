"""Small Mufevik configurations and random weights for the tests, and an error measure.

The configurations differ from one another in every size, in the order of the layers and in what is left out (the
residual streams, the groups of experts, the shared expert, a layer's feed-forward, the rotation); values that a given
checkpoint might happen to make equal (key and value sizes of a head, query and key-value head counts, the head sizes
of the two mixers of a layer) or 1 are unequal here, or 1 where a checkpoint would have more.  Weights are rounded to
bfloat16 so that both precisions read the same values.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List

import torch

NAME = "Mufevik"


def _left(heads, kv, dim, vdim, scale, rot=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return m


def _moe(experts, top, ff, groups=None, shared=None):
    r = {"experts": experts, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "router": r, "expert": {"ff": ff}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def config_a() -> dict:
    """Three streams; grouped heads on both kinds of mixer; a rotation of part of a head; groups of experts."""
    return {"architecture": NAME, "vocab": 211, "width": 96, "streams": 3, "logit_scale": 0.7, "norm": {"eps": 1e-5},
            "layers": [
                {"type": "parallel", "mixer": {"left": _left(4, 2, 24, 40, 0.2, (16, 5000.0)),
                                                "right": {"heads": 3, "dim": 20, "vdim": 24, "tau": 7.0}},
                 "mlp": _moe(8, 2, 40, groups=(4, 2), shared=56)},
                {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 24, "vdim": 16, "conv": 3},
                 "mlp": _moe(6, 3, 32)},
                {"type": "parallel", "mixer": {"left": _left(2, 2, 16, 8, 0.3), "right": {"heads": 2, "dim": 8, "vdim": 40, "tau": 3.0}},
                 "mlp": None},
            ]}


def config_b() -> dict:
    """One plain residual stream (no ``streams`` key); a delta layer first; convolutions of two and five taps; one head."""
    return {"architecture": NAME, "vocab": 130, "width": 64, "logit_scale": 1.0, "norm": {"eps": 1e-3},
            "layers": [
                {"type": "delta", "mixer": {"heads": 1, "kv_heads": 1, "dim": 40, "vdim": 72, "conv": 2}, "mlp": _moe(4, 1, 24, shared=16)},
                {"type": "parallel", "mixer": {"left": _left(1, 1, 32, 16, 0.18, (32, 100.0)),
                                                "right": {"heads": 1, "dim": 72, "vdim": 16, "tau": 1.0}},
                 "mlp": _moe(5, 5, 16, groups=(1, 1))},
                {"type": "delta", "mixer": {"heads": 6, "kv_heads": 3, "dim": 8, "vdim": 8, "conv": 5}, "mlp": None},
            ]}


def config_c() -> dict:
    """A single stream that still goes through hyper-connections (``streams``: 1); a convolution of one tap."""
    return {"architecture": NAME, "vocab": 97, "width": 32, "streams": 1, "logit_scale": 2.0, "norm": {"eps": 1e-6},
            "layers": [
                {"type": "parallel", "mixer": {"left": _left(6, 3, 8, 12, 0.35, (4, 30000.0)),
                                                "right": {"heads": 2, "dim": 12, "vdim": 8, "tau": 30.0}},
                 "mlp": _moe(6, 2, 24, groups=(3, 1))},
                {"type": "delta", "mixer": {"heads": 2, "kv_heads": 2, "dim": 16, "vdim": 24, "conv": 1}, "mlp": _moe(3, 2, 8, shared=8)},
            ]}


def config_d() -> dict:
    """Sizes that fit no kernel's favourite multiple: a width of 100, five heads of 12 with values of 36, a rotation of six
    dimensions, nine experts in three groups, feed-forwards of 20, seven streams."""
    return {"architecture": NAME, "vocab": 77, "width": 100, "streams": 7, "logit_scale": 0.4, "norm": {"eps": 1e-4},
            "layers": [
                {"type": "delta", "mixer": {"heads": 3, "kv_heads": 1, "dim": 20, "vdim": 44, "conv": 4}, "mlp": _moe(9, 2, 20, groups=(3, 1), shared=12)},
                {"type": "parallel", "mixer": {"left": _left(5, 5, 12, 36, 0.25, (6, 777.0)),
                                                "right": {"heads": 5, "dim": 36, "vdim": 12, "tau": 11.0}},
                 "mlp": _moe(9, 4, 20, groups=(3, 2))},
            ]}


CONFIGS = {"a": config_a, "b": config_b, "c": config_c, "d": config_d}
DECAY_RANK = 8          # rows of the decay's first projection: only the tensor's shape gives it


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    W, S, out = cfg["width"], cfg.get("streams"), {}
    out["embed"] = (cfg["vocab"], W)
    out["head"] = (cfg["vocab"], W)
    out["final.norm"] = ()
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        for n in ["1"] + (["2"] if layer["mlp"] else []):
            out[p + "norm" + n] = ()
            if S:
                out.update({f"{p}hc{n}.in": (S,), f"{p}hc{n}.out": (S,), f"{p}hc{n}.mix": (S, S)})
        if layer["type"] == "parallel":
            l, r = m["left"], m["right"]
            out.update({p + "mix.left.q": (l["heads"] * l["dim"], W), p + "mix.left.k": (l["kv_heads"] * l["dim"], W),
                        p + "mix.left.v": (l["kv_heads"] * l["vdim"], W), p + "mix.left.o": (W, l["heads"] * l["vdim"]),
                        p + "mix.left.temp": (l["heads"],), p + "mix.left.talk": (l["heads"], l["heads"]),
                        p + "mix.left.out": (W,), p + "mix.right.out": (W,),
                        p + "mix.right.q": (r["heads"] * r["dim"], W), p + "mix.right.k": (r["heads"] * r["dim"], W),
                        p + "mix.right.v": (r["heads"] * r["vdim"], W), p + "mix.right.g": (r["heads"] * r["vdim"], W),
                        p + "mix.right.o": (W, r["heads"] * r["vdim"]), p + "mix.right.norm": (r["vdim"],),
                        p + "mix.right.a1": (DECAY_RANK, W), p + "mix.right.a2": (r["heads"] * r["dim"], DECAY_RANK),
                        p + "mix.right.a2.b": (r["heads"] * r["dim"],)})
        else:
            H, G, d, dv, K = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            out.update({p + "mix.q": (G * d, W), p + "mix.q.conv": (G * d, K), p + "mix.k": (G * d, W), p + "mix.k.conv": (G * d, K),
                        p + "mix.v": (H * dv, W), p + "mix.v.conv": (H * dv, K), p + "mix.b": (H, W), p + "mix.a": (H, W),
                        p + "mix.A_log": (H,), p + "mix.dt_bias": (H,), p + "mix.g": (H * dv, W), p + "mix.o": (W, H * dv),
                        p + "mix.norm": (dv,)})
        if layer["mlp"]:
            mlp = layer["mlp"]
            ff = mlp["expert"]["ff"]
            for e in range(mlp["router"]["experts"]):
                out.update({f"{p}mlp.e{e}.gate": (ff, W), f"{p}mlp.e{e}.up": (ff, W), f"{p}mlp.e{e}.down": (W, ff)})
            out.update({p + "mlp.router": (mlp["router"]["experts"], W), p + "mlp.correction": (mlp["router"]["experts"],)})
            if mlp.get("shared"):
                sf = mlp["shared"]["ff"]
                out.update({p + "mlp.shared.gate": (sf, W), p + "mlp.shared.up": (sf, W), p + "mlp.shared.down": (W, sf),
                            p + "mlp.shared.sg": (1, W)})
    return out


def random_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if name.endswith(".conv"):
            t = torch.randn(shape, generator=g) * 0.6
        elif last == "talk" or (last == "mix" and ".hc" in name):
            t = torch.eye(shape[0]) + 0.3 * torch.randn(shape, generator=g)
        elif last == "in":
            t = 1.0 / shape[0] + 0.2 * torch.randn(shape, generator=g)
        elif last == "router":
            t = torch.randn(shape, generator=g) * (2.5 / shape[1] ** 0.5)
        elif last == "correction":
            t = torch.randn(shape, generator=g) * 0.1 - 0.2           # choice scores are often negative
        elif last in ("A_log", "dt_bias"):
            t = torch.randn(shape, generator=g) * 0.7
        elif name.endswith("a2.b"):
            t = 2.0 + torch.randn(shape, generator=g)
        elif len(shape) == 2:
            t = torch.randn(shape, generator=g) * (1.4 / shape[1] ** 0.5)
        else:
            t = 1.0 + 0.25 * torch.randn(shape, generator=g)          # norm weights and gains, temperatures, output weights
        out[name] = t.to(torch.bfloat16)
    return out


def write_folder(cfg: dict, weights: Dict[str, torch.Tensor], out_dir: str) -> str:
    from cpmcu_b200.weights.safetensors_io import save_file

    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(out_dir, "model.safetensors"))
    return out_dir


def random_ids(vocab: int, n: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def moe_layers(cfg: dict) -> int:
    return sum(1 for layer in cfg["layers"] if layer["mlp"])


# Largest allowed root mean square of (engine - plain) over the vocabulary, the mean difference taken off, relative to
# the root mean square of the plain logits, for the worst row and for the median row.  float32: summation order only.
# bfloat16: activations between the kernels and the cached keys and values are rounded to bfloat16 in the engine; with
# these weights (sharp routers, head mixes and stream mixes far from the identity) single rows react strongly to that
# rounding, so the worst row has a loose bound and the median a tight one, and float32 carries the exact comparison (there
# too a single row of a sequence can be 100 times less exact than the median, whatever the schedule).
TOL = {"float32": 5e-4, "bfloat16": 0.6}
MEDIAN_TOL = {"float32": 2e-5, "bfloat16": 4e-2}
# A token's choice of experts may fall the other way where two choice scores nearly tie; the plain implementation uses
# the engine's choice, which must lie this close to the rule's cut-off (scores are in [0, 1])
CHOICE_SLACK = {"float32": 1e-5, "bfloat16": 4e-2}


def row_errors(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert got.shape == want.shape, (got.shape, want.shape)
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()
