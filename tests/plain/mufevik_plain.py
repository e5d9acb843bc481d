"""A plain, slow implementation of the Mufevik architecture on whole sequences: no cache, no state carried
between calls, one function per mechanism, float64 by default.  It shares no code with the package; it reads
the raw configuration dictionary and the tensors by their names in the checkpoint.

Notation: T tokens, W the model's width, S residual streams; x [T, S, W] (S = 1 without hyper-connections).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch

DT = torch.float64


def scalar_rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) times one number."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * gain


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def rotate(x: torch.Tensor, dims: int, base: float, first: int = 0) -> torch.Tensor:
    """x [T, heads, d]: pairs (i, i + dims/2) of the first ``dims`` columns turned by p * base^(-2i/dims)."""
    if not dims:
        return x
    T = x.shape[0]
    half = dims // 2
    p = torch.arange(first, first + T, dtype=DT)
    f = torch.pow(torch.tensor(float(base), dtype=DT), -2.0 * torch.arange(half, dtype=DT) / dims)
    a = p[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def talking_softmax_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict) -> torch.Tensor:
    """Causal softmax attention whose weights are mixed across heads after the softmax."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, d)
    k = (h @ w[p + "k"].T).view(T, G, d)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    rot = m.get("rot")
    if rot:
        q, k = rotate(q, rot["dims"], rot["base"]), rotate(k, rot["dims"], rot["base"])
    rep = H // G
    visible = torch.tril(torch.ones(T, T, dtype=torch.bool))
    weights = []
    for g in range(H):
        s = (q[:, g] @ k[:, g // rep].T) * m["scale"] * w[p + "temp"][g]
        s = s.masked_fill(~visible, float("-inf"))
        weights.append(torch.softmax(s, dim=-1))
    weights = torch.stack(weights)                                     # [H, T, T]
    mixed = torch.einsum("hg,gij->hij", w[p + "talk"], weights)
    out = torch.stack([mixed[hh] @ v[:, hh // rep] for hh in range(H)], dim=1)       # [T, H, dv]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def matrix_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor,
                      beta: Optional[torch.Tensor] = None, state: Optional[torch.Tensor] = None):
    """q, k [T, H, d], v [T, H, dv], decay [T, H, d] or [T, H, 1], beta [T, H] or None (no delta correction).
    S <- diag(decay) S; u = v or beta (v - S^T k); S <- S + k u^T; o = S^T q.  Returns (o [T, H, dv], last S)."""
    T, H, d = q.shape
    S = torch.zeros(H, d, v.shape[-1], dtype=q.dtype) if state is None else state.clone()
    out = torch.empty(T, H, v.shape[-1], dtype=q.dtype)
    for t in range(T):
        S = decay[t][:, :, None] * S
        u = v[t] if beta is None else beta[t][:, None] * (v[t] - torch.einsum("hcv,hc->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out[t] = torch.einsum("hcv,hc->hv", S, q[t])
    return out, S


def gated_linear_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Per head S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, alpha = sigmoid(z)^(1/tau) per key channel."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, d)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = torch.pow(torch.sigmoid(z), 1.0 / m["tau"]).view(T, H, d)
    out, _ = matrix_recurrence(q, k, v, alpha)
    out = rms_norm(out, w[p + "norm"], eps).reshape(T, H * dv)
    return (out * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def parallel_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    a = talking_softmax_attention(h, w, p + "left.", m["left"])
    b = gated_linear_attention(h, w, p + "right.", m["right"], eps)
    return 0.5 * (rms_norm(a, w[p + "left.out"], eps) + rms_norm(b, w[p + "right.out"], eps))


def short_convolution(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, K]: y_t = sum_j taps[:, K-1-j] x_(t-j), zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(K):
        y = y + padded[j:j + T] * taps[:, j]
    return y


def gated_delta_rule(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_convolution(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, d)
    k = silu(short_convolution(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, d)
    v = silu(short_convolution(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                                   # [T, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * torch.nn.functional.softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    rep = H // G
    out, _ = matrix_recurrence(q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1), v, decay[:, :, None], beta)
    out = rms_norm(out, w[p + "norm"], eps).reshape(T, H * dv)
    return (out * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def gated_expert(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route_scores(z: torch.Tensor, correction: torch.Tensor, r: dict):
    """Router logits z [T, E] -> (scores s, choice scores with the experts of groups that are not kept at -inf)."""
    E = r["experts"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    s = torch.softmax(z, dim=-1)
    choice = s + correction
    per = E // groups["count"]
    best = choice.view(-1, groups["count"], per).max(-1).values
    kept = best.topk(groups["keep"], dim=-1).indices
    allowed = torch.zeros(z.shape[0], groups["count"], dtype=torch.bool)
    allowed.scatter_(1, kept, True)
    return s, choice.masked_fill(~allowed.repeat_interleave(per, dim=1), float("-inf"))


def route(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, r: dict):
    """(chosen experts [T, top], their weights [T, top]): softmax scores, choice by score + correction among the
    experts of the best groups, weights the plain scores of the chosen."""
    s, choice = route_scores(h @ w[p + "router"].T, w[p + "correction"], r)
    chosen = choice.topk(r["top"], dim=-1).indices
    return chosen, torch.gather(s, 1, chosen)


def choice_slack(raw: torch.Tensor, forced: torch.Tensor, r: dict) -> List[float]:
    """How far a given choice of experts lies from the rule's, per token: the larger of (the lowest kept group's score
    minus the lowest score of a group the choice uses) and (the rule's cut-off among the experts of the groups the
    choice uses, completed by the best others, minus the lowest chosen choice score); 0 when the choice is the rule's."""
    groups = r.get("groups") or {"count": 1, "keep": 1}
    count, keep, top = groups["count"], groups["keep"], r["top"]
    per = r["experts"] // count
    out = []
    for t in range(raw.shape[0]):
        gbest = raw[t].view(count, per).max(-1).values
        order = gbest.argsort(descending=True).tolist()
        used = sorted(set((forced[t] // per).tolist()))
        g_slack = max(0.0, float(gbest[order[keep - 1]] - min(gbest[g] for g in used)))
        for g in order:
            if len(used) >= keep:
                break
            if g not in used:
                used.append(g)
        mask = torch.full_like(raw[t], float("-inf"))
        for g in used:
            mask[g * per:(g + 1) * per] = 0.0
        cut = (raw[t] + mask).topk(top).values.min()
        out.append(max(g_slack, float(cut - raw[t][forced[t]].min()), 0.0) if len(used) <= keep else float("inf"))
    return out


def mixture_of_experts(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: dict,
                       forced: Optional[torch.Tensor] = None, slack: Optional[List[float]] = None) -> torch.Tensor:
    """``forced`` [T, top]: experts to use instead of the rule's own choice (the weights stay the scores s); ``slack``
    then receives, per token, how far the lowest forced choice score lies below the rule's cut-off (0: the rule's choice)."""
    chosen, weight = route(h, w, p, mlp["router"])
    if forced is not None:
        forced = forced.long()
        s, _ = route_scores(h @ w[p + "router"].T, w[p + "correction"], mlp["router"])
        if slack is not None:
            slack.extend(choice_slack(s + w[p + "correction"], forced, mlp["router"]))
        chosen, weight = forced, torch.gather(s, 1, forced)
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weight[t]):
            out[t] += g * gated_expert(h[t:t + 1], w, f"{p}e{e}.")[0]
    if mlp.get("shared"):
        out = out + torch.sigmoid(h @ w[p + "shared.sg"].T) * gated_expert(h, w, p + "shared.")
    return out


def hyper_read(x: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    """x [T, S, W] -> sum_s in[s] x_s."""
    return torch.einsum("s,tsw->tw", w[p + "in"], x)


def hyper_write(x: torch.Tensor, y: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    """x_t <- sum_s mix[s, t] x_s + out[t] y, all streams from the old ones."""
    return torch.einsum("sr,tsw->trw", w[p + "mix"], x) + w[p + "out"][None, :, None] * y[:, None, :]


def mixer(h, w, p, layer, eps):
    if layer["type"] == "parallel":
        return parallel_mixer(h, w, p, layer["mixer"], eps)
    if layer["type"] == "delta":
        return gated_delta_rule(h, w, p, layer["mixer"], eps)
    raise ValueError(layer["type"])


def forward(config: dict, weights: Dict[str, torch.Tensor], ids: Sequence[int], collect: Optional[List[torch.Tensor]] = None,
            forced: Optional[List[torch.Tensor]] = None, slack: Optional[List[float]] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  ``collect`` receives the residual stream (the sum of the streams)
    after every layer.  ``forced``: per layer with a mixture of experts (in order), the experts [T, top] to use."""
    forced = list(forced) if forced is not None else None
    w = {k: (v.to(DT) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    hyper = "streams" in config
    S = config.get("streams", 1)
    e = w["embed"][list(ids)]
    x = e[:, None, :].repeat(1, S, 1)
    for i, layer in enumerate(config["layers"]):
        L = f"l{i}."
        subs = [("1", lambda hh: mixer(hh, w, L + "mix.", layer, eps))]
        if layer.get("mlp"):
            f = forced.pop(0) if forced else None
            subs.append(("2", lambda hh, f=f: mixture_of_experts(hh, w, L + "mlp.", layer["mlp"], f, slack)))
        for n, fn in subs:
            if hyper:
                u = hyper_read(x, w, f"{L}hc{n}.")
                x = hyper_write(x, fn(scalar_rms_norm(u, w[f"{L}norm{n}"], eps)), w, f"{L}hc{n}.")
            else:
                x = x + fn(scalar_rms_norm(x[:, 0], w[f"{L}norm{n}"], eps))[:, None, :]
        if collect is not None:
            collect.append(x.sum(1))
    y = scalar_rms_norm(x.sum(1), w["final.norm"], eps)
    return (y @ w["head"].T) * config.get("logit_scale", 1.0)


def greedy(config: dict, weights: Dict[str, torch.Tensor], prompt: Sequence[int], n_new: int):
    """(tokens, gaps): the ``n_new`` tokens greedy decoding appends, and at each the gap between the two best logits."""
    ids, tokens, gaps = list(prompt), [], []
    for _ in range(n_new):
        last = forward(config, weights, ids)[-1]
        best = torch.topk(last, 2)
        tokens.append(int(best.indices[0]))
        gaps.append(float(best.values[0] - best.values[1]))
        ids.append(tokens[-1])
    return tokens, gaps
