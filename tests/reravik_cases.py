"""Small Reravik configurations and random weights for the tests, and an error measure.

The configurations differ from one another in every size, in the order of the layers, in the repeated group
and in the windows; several values that a given checkpoint might happen to make equal (query and value sizes of a
head, the ranks of the two latents, the widths of the recurrent layers) or 1 (heads, passes) are unequal here, or 1
where a checkpoint would have more.  Weights are rounded to bfloat16 so that both precisions read the same values.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Sequence

import torch

NAME = "Reravik"


def _latent(heads, dim, vdim, q_rank, kv_rank, scale, window):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    return m


def config_a() -> dict:
    """Four layers, the middle two run three times; windows of 37 (inside a page) and 70 (across a page border)."""
    return {"architecture": NAME, "vocab": 211, "width": 96, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
            "layers": [
                {"type": "mingru", "mixer": {"width": 80}, "mlp": {"kind": "dense", "ff": 112}},
                {"type": "latent_attention", "mixer": _latent(3, 16, 24, 40, 48, 0.21, 37), "mlp": {"kind": "dense", "ff": 64}},
                {"type": "mingru", "mixer": {"width": 72}, "mlp": None},
                {"type": "latent_attention", "mixer": _latent(2, 32, 16, 24, 64, 0.3, 70), "mlp": {"kind": "dense", "ff": 112}},
            ],
            "loop": {"start": 1, "stop": 3, "times": 3}}


def config_b() -> dict:
    """One head, no window, a latent rank that is no multiple of 32, a single pass over a group of one layer, an
    attention layer first and without a feed-forward."""
    return {"architecture": NAME, "vocab": 130, "width": 64, "embedding": {"scale": 1.5}, "norm": {"eps": 1e-3},
            "layers": [
                {"type": "latent_attention", "mixer": _latent(1, 24, 40, 56, 72, 0.17, None), "mlp": None},
                {"type": "mingru", "mixer": {"width": 96}, "mlp": {"kind": "dense", "ff": 48}},
                {"type": "latent_attention", "mixer": _latent(5, 8, 8, 16, 32, 0.4, 3), "mlp": {"kind": "dense", "ff": 80}},
            ],
            "loop": {"start": 0, "stop": 1, "times": 1}}


def config_c() -> dict:
    """No repeated group at all; a window of one token (a query sees itself only) and a window of two."""
    return {"architecture": NAME, "vocab": 97, "width": 32, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-6},
            "layers": [
                {"type": "latent_attention", "mixer": _latent(2, 16, 16, 16, 16, 0.25, 1), "mlp": {"kind": "dense", "ff": 40}},
                {"type": "latent_attention", "mixer": _latent(4, 8, 12, 20, 24, 0.35, 2), "mlp": None},
                {"type": "mingru", "mixer": {"width": 32}, "mlp": {"kind": "dense", "ff": 24}},
            ]}


def config_d() -> dict:
    """Sizes that fit no kernel's favourite multiple: a width of 100, ranks of 50 and 40, seven heads of 20 with values
    of 12, a recurrent width of 36, a feed-forward of 52, a window of five, one layer run four times."""
    return {"architecture": NAME, "vocab": 77, "width": 100, "embedding": {"scale": 7.0}, "norm": {"eps": 1e-4},
            "layers": [
                {"type": "mingru", "mixer": {"width": 36}, "mlp": {"kind": "dense", "ff": 52}},
                {"type": "latent_attention", "mixer": _latent(7, 20, 12, 50, 40, 0.22, 5), "mlp": {"kind": "dense", "ff": 52}},
                {"type": "mingru", "mixer": {"width": 44}, "mlp": None},
            ],
            "loop": {"start": 1, "stop": 2, "times": 4}}


CONFIGS = {"a": config_a, "b": config_b, "c": config_c, "d": config_d}


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    W, out = cfg["width"], {}
    out["embed"] = (cfg["vocab"], W)
    out["head"] = (cfg["vocab"], W)
    out["final.norm"] = (W,)
    out["final.norm.b"] = (W,)
    if cfg.get("loop"):
        out["loop.step"] = (cfg["loop"]["times"], W)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        norms = ["norm1", "norm1b"] + (["norm2", "norm2b"] if layer["mlp"] else [])
        for n in norms:
            out[p + n] = (W,)
            out[p + n + ".b"] = (W,)
        out[p + "shift"] = (W,)
        if layer["type"] == "mingru":
            w = m["width"]
            out.update({p + "mix.z": (w, W), p + "mix.z.b": (w,), p + "mix.x": (w, W), p + "mix.x.b": (w,),
                        p + "mix.g": (w, W), p + "mix.o": (W, w)})
        else:
            H = m["heads"]
            out.update({p + "mix.dq": (m["q_rank"], W), p + "mix.dq.norm": (m["q_rank"],), p + "mix.uq": (H * m["dim"], m["q_rank"]),
                        p + "mix.dkv": (m["kv_rank"], W), p + "mix.dkv.norm": (m["kv_rank"],),
                        p + "mix.uk": (H * m["dim"], m["kv_rank"]), p + "mix.uv": (H * m["vdim"], m["kv_rank"]),
                        p + "mix.o": (W, H * m["vdim"])})
        if layer["mlp"]:
            ff = layer["mlp"]["ff"]
            out.update({p + "mlp.gate": (ff, W), p + "mlp.up": (ff, W), p + "mlp.down": (W, ff)})
    return out


def random_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if len(shape) == 2 and name != "loop.step":
            t = torch.randn(shape, generator=g) * (1.4 / shape[1] ** 0.5)
        elif name.endswith("shift"):
            t = torch.rand(shape, generator=g)
        elif name.endswith(".b") or name == "loop.step":
            t = torch.randn(shape, generator=g) * 0.3
        else:
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
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


# Largest allowed root mean square of (engine - plain) over the vocabulary, the mean difference taken off, relative to
# the root mean square of the plain logits.  float32: summation order only.  bfloat16: activations between the kernels
# and the cached latents are rounded to bfloat16 in the engine.
TOL = {"float32": 3e-5, "bfloat16": 3e-2}


def row_errors(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert got.shape == want.shape, (got.shape, want.shape)
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()
