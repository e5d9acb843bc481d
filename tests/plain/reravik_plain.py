"""A plain, slow implementation of the Reravik architecture on whole sequences: no cache, no state carried
between calls, one function per mechanism, float64 by default.  It shares no code with the package; it reads
the raw configuration dictionary and the tensors by their names in the checkpoint.

Notation: T tokens, W the model's width, x the residual stream [T, W].
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch

DT = torch.float64


def position_vectors(n_tokens: int, width: int, first: int = 0) -> torch.Tensor:
    """[T, W]: column 2i holds sin(p f_i), column 2i+1 cos(p f_i), f_i = 10000^(-2i/W), p counted from ``first``."""
    p = torch.arange(first, first + n_tokens, dtype=DT)
    i = torch.arange(width // 2, dtype=DT)
    angle = p[:, None] * torch.pow(torch.tensor(10000.0, dtype=DT), -2.0 * i / width)[None, :]
    out = torch.empty(n_tokens, width, dtype=DT)
    out[:, 0::2] = torch.sin(angle)
    out[:, 1::2] = torch.cos(angle)
    return out


def embed(ids: Sequence[int], table: torch.Tensor, scale: float) -> torch.Tensor:
    return table[list(ids)] * scale + position_vectors(len(ids), table.shape[1])


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * weight + bias


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def token_shift(h: torch.Tensor, mix: torch.Tensor) -> torch.Tensor:
    """h_t + (h_{t-1} - h_t) * mix with zeros before the first token."""
    before = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)
    return h + (before - h) * mix


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def dense_mlp(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    return (gelu_tanh(h @ w[prefix + "gate"].T) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def min_gru(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    z = torch.sigmoid(h @ w[prefix + "z"].T + w[prefix + "z.b"])
    u = h @ w[prefix + "x"].T + w[prefix + "x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    state = torch.zeros(z.shape[1], dtype=h.dtype)
    states = []
    for t in range(h.shape[0]):
        state = (1.0 - z[t]) * state + z[t] * cand[t]
        states.append(state)
    g = h @ w[prefix + "g"].T
    return (torch.stack(states) * (g * torch.sigmoid(g))) @ w[prefix + "o"].T


def visible(n_tokens: int, window: Optional[int]) -> torch.Tensor:
    """[T, T] bool: query i sees key j iff 0 <= i - j (< window when there is one)."""
    i = torch.arange(n_tokens)[:, None]
    j = torch.arange(n_tokens)[None, :]
    ok = i >= j
    if window is not None:
        ok &= (i - j) < window
    return ok


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, mixer: dict, eps: float,
                     probabilities: Optional[list] = None) -> torch.Tensor:
    T = h.shape[0]
    H, d, vd = mixer["heads"], mixer["dim"], mixer["vdim"]
    q = (rms_norm(h @ w[prefix + "dq"].T, w[prefix + "dq.norm"], eps) @ w[prefix + "uq"].T).view(T, H, d)
    c = rms_norm(h @ w[prefix + "dkv"].T, w[prefix + "dkv.norm"], eps)
    k = (c @ w[prefix + "uk"].T).view(T, H, d)
    v = (c @ w[prefix + "uv"].T).view(T, H, vd)
    window = (mixer.get("mask") or {}).get("size")
    scores = torch.einsum("ihd,jhd->hij", q, k) * mixer["scale"]
    scores = scores.masked_fill(~visible(T, window), float("-inf"))
    p = torch.softmax(scores, dim=-1)
    if probabilities is not None:
        probabilities.append(p)
    return torch.einsum("hij,jhd->ihd", p, v).reshape(T, H * vd) @ w[prefix + "o"].T


def run_order(cfg: dict) -> List[Tuple[int, Optional[int]]]:
    """(layer, pass number if a pass through the repeated group begins here)."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    order: List[Tuple[int, Optional[int]]] = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg: dict, weights: Dict[str, torch.Tensor], ids: Sequence[int], streams: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence; ``streams`` receives the residual stream after every run of a layer."""
    w = {k: v.to(DT) for k, v in weights.items() if v.is_floating_point()}
    eps = cfg["norm"]["eps"]
    x = embed(ids, w["embed"], cfg["embedding"]["scale"])
    embedded = x.clone()
    for layer, enters in run_order(cfg):
        if enters is not None:
            if enters > 0:
                x = x + embedded
            x = x + w["loop.step"][enters]
        spec, pre = cfg["layers"][layer], f"l{layer}."
        h = token_shift(layer_norm(x, w[pre + "norm1"], w[pre + "norm1.b"], eps), w[pre + "shift"])
        if spec["type"] == "mingru":
            a = min_gru(h, w, pre + "mix.")
        elif spec["type"] == "latent_attention":
            a = latent_attention(h, w, pre + "mix.", spec["mixer"], eps)
        else:
            raise ValueError(spec["type"])
        x = x + layer_norm(a, w[pre + "norm1b"], w[pre + "norm1b.b"], eps)
        if spec.get("mlp") is not None:
            f = dense_mlp(layer_norm(x, w[pre + "norm2"], w[pre + "norm2.b"], eps), w, pre + "mlp.")
            x = x + layer_norm(f, w[pre + "norm2b"], w[pre + "norm2b.b"], eps)
        if streams is not None:
            streams.append(x.clone())
    return layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T


def greedy(cfg: dict, weights: Dict[str, torch.Tensor], prompt: Sequence[int], n_new: int) -> Tuple[List[int], List[float]]:
    """(tokens, per token the gap between the two best logits) of greedy generation, lowest index on ties."""
    ids, out, gaps = list(prompt), [], []
    for _ in range(n_new):
        last = forward(cfg, weights, ids)[-1]
        top = last.topk(2).values
        gaps.append(float(top[0] - top[1]))
        tok = int((last == last.max()).nonzero()[0])
        out.append(tok)
        ids.append(tok)
    return out, gaps
